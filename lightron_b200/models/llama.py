"""Llama-style decoder with the reference's parameter names and math.

Parity: ``model/model.py`` of the reference: pre-norm block ``h = x + attn(norm(x)); out = h +
ffn(norm(h))`` (``:228-231``), SwiGLU MLP ``w2(silu(w1 x) * w3 x)`` (``:50-69``), GQA attention
with interleaved-pair RoPE and causal softmax (``:119-202``), untied embedding / output head and a
final RMSNorm (``:234-271``).  state_dict keys are identical: ``tok_embeddings.weight``,
``layers.{i}.attention.{wq,wk,wv,wo}.weight``, ``layers.{i}.feed_forward.{w1,w3,w2}.weight``,
``layers.{i}.{attention_norm,ffn_norm}.weight``, ``norm.weight``, ``output.weight`` and for MoE layers
``layers.{i}.feed_forward.gate.weight`` / ``.experts.{e}.{w1,w3,w2}.weight``.

What is different by design:
* activations are kept as one flattened ``[tokens, hidden]`` matrix, the natural operand of the
  TMA-fed GEMM kernels; under sequence parallelism its rows are sharded across the TP group;
* q/k/v (and gate/up) projections are one GEMM over row-adjacent weights living in a flat
  parameter arena, RoPE + attention consume the fused projection output in place, and each
  residual add is fused with the RMSNorm that follows it;
* GQA works (the reference views k/v with the query head count, ``:166-167``), any sequence
  length up to ``max_seq_len`` works, and the RoPE table is a real fp32 cos/sin pair so that a
  bf16 cast cannot drop its imaginary part;
* a pipeline stage builds only its own layers (``layer_range``) instead of the whole model;
* the head feeds a vocab-parallel cross-entropy (``loss``) instead of all-gathering logits; the
  full-logits ``forward`` is kept for API parity.
"""
from __future__ import annotations

import zlib
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from .. import mesh as _mesh
from ..config import ModelArgs
from ..ops import functional as OF
from ..ops import reference as ref
from ..parallel import comm, fused
from ..parallel.tp import ColumnParallelLinear, Linear, RowParallelLinear, VocabParallelEmbedding


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x):
        return OF.rmsnorm(x, self.weight, self.eps)


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, dim: int, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_embeddings, dim, dtype=dtype, device=device))

    def forward(self, tokens):
        return OF.embedding(tokens, self.weight, 0)


def _col(args: ModelArgs, i, o, ctx, **kw):
    if args.tp_size > 1:
        return ColumnParallelLinear(i, o, bias=False, group=ctx.tp_group, sequence_parallel=args.sequence_parallel, **kw)
    return Linear(i, o, **kw)


def _row(args: ModelArgs, i, o, ctx, **kw):
    if args.tp_size > 1:
        return RowParallelLinear(i, o, bias=False, group=ctx.tp_group, sequence_parallel=args.sequence_parallel, **kw)
    return Linear(i, o, **kw)


class MLP(nn.Module):
    def __init__(self, args: ModelArgs, ctx, **kw):
        super().__init__()
        hidden = args.ffn_hidden
        self.tp_group = ctx.tp_group if args.tp_size > 1 else None
        self.sp = args.sequence_parallel and args.tp_size > 1
        self.w1 = _col(args, args.dim, hidden, ctx, **kw)     # gate
        self.w3 = _col(args, args.dim, hidden, ctx, **kw)     # up
        self.w2 = _row(args, hidden, args.dim, ctx, **kw)     # down

    def forward(self, x: torch.Tensor, sp: Optional[bool] = None) -> torch.Tensor:
        sp = self.sp if sp is None else sp
        if self.tp_group is None:
            return OF.swiglu_mlp(x, self.w1.weight, self.w3.weight, self.w2.weight)
        if sp:
            gu = fused.all_gather_linear(x, (self.w1.weight, self.w3.weight), self.tp_group)
        else:
            gu = OF.linear(comm.copy_to_group(x, self.tp_group), self.w1.weight, self.w3.weight)
        a = OF.swiglu(gu)
        if sp:
            return fused.linear_reduce_scatter(a, self.w2.weight, self.tp_group)
        return comm.reduce_from_group(OF.linear(a, self.w2.weight), self.tp_group)


class Attention(nn.Module):
    def __init__(self, args: ModelArgs, ctx, **kw):
        super().__init__()
        tp = args.tp_size
        assert args.n_heads % tp == 0, f"n_heads ({args.n_heads}) must be divisible by tp_size ({tp})"
        assert args.n_kv_heads % tp == 0, f"n_kv_heads ({args.n_kv_heads}) must be divisible by tp_size ({tp})"
        self.n_heads = args.n_heads // tp
        self.n_kv_heads = args.n_kv_heads // tp
        self.head_dim = args.head_dim
        self.n_rep = self.n_heads // self.n_kv_heads
        self.tp_group = ctx.tp_group if tp > 1 else None
        self.cp_group = ctx.cp_group if args.cp_size > 1 else None
        self.cp_mode = args.cp_mode
        self.sp = args.sequence_parallel and tp > 1
        d = self.head_dim
        self.wq = _col(args, args.dim, args.n_heads * d, ctx, **kw)
        self.wk = _col(args, args.dim, args.n_kv_heads * d, ctx, **kw)
        self.wv = _col(args, args.dim, args.n_kv_heads * d, ctx, **kw)
        self.wo = _row(args, args.n_heads * d, args.dim, ctx, **kw)

    def forward(self, x: torch.Tensor, B: int, S: int, cos, sin, positions) -> torch.Tensor:
        """x [T(/tp if SP), H] -> [T(/tp), H]; T = B*S with S the local (per-CP-rank) length."""
        if self.sp:
            qkv = fused.all_gather_linear(x, (self.wq.weight, self.wk.weight, self.wv.weight), self.tp_group)
        else:
            qkv = OF.linear(comm.copy_to_group(x, self.tp_group), self.wq.weight, self.wk.weight, self.wv.weight)
        hq, hkv, d = self.n_heads, self.n_kv_heads, self.head_dim
        if self.cp_group is None:
            o = OF.rope_attention_qkv(qkv, cos, sin, positions, B, S, hq, hkv, d)
        else:
            from ..parallel import cp
            o = cp.context_parallel_attention(qkv, cos, sin, positions, B, S, hq, hkv, d, self.cp_group, self.cp_mode)
        if self.sp:
            return fused.linear_reduce_scatter(o, self.wo.weight, self.tp_group)
        return comm.reduce_from_group(OF.linear(o, self.wo.weight), self.tp_group)


class TransformerBlock(nn.Module):
    def __init__(self, args: ModelArgs, layer_id: int, ctx, **kw):
        super().__init__()
        self.layer_id = layer_id
        self.attention = Attention(args, ctx, **kw)
        if args.is_moe_layer(layer_id):
            from .moe import MoEFeedForward
            self.feed_forward = MoEFeedForward(args, ctx, **kw)
        else:
            self.feed_forward = MLP(args, ctx, **kw)
        self.attention_norm = RMSNorm(args.dim, eps=args.norm_eps, **kw)
        self.ffn_norm = RMSNorm(args.dim, eps=args.norm_eps, **kw)

    def forward(self, h, delta, B, S, cos, sin, positions):
        """Carries the residual stream as (h, delta) with h + delta pending, so that each add is
        fused with the following norm.  Returns the next (h, delta)."""
        if delta is None:
            x = OF.rmsnorm(h, self.attention_norm.weight, self.attention_norm.eps)
        else:
            h, x = OF.add_rmsnorm(delta, h, self.attention_norm.weight, self.attention_norm.eps)
        a = self.attention(x, B, S, cos, sin, positions)
        h, x = OF.add_rmsnorm(a, h, self.ffn_norm.weight, self.ffn_norm.eps)
        f = self.feed_forward(x)
        return h, f


class LightronTransformer(nn.Module):
    def __init__(self, args: ModelArgs, ctx: Optional[_mesh.ParallelContext] = None,
                 layer_range: Optional[Tuple[int, int]] = None, first_stage: bool = True, last_stage: bool = True,
                 dtype=None, device=None):
        super().__init__()
        self.args = args
        self.ctx = ctx if ctx is not None else _mesh.get_context()
        ctx = self.ctx
        kw = dict(dtype=dtype, device=device)
        self.first_stage, self.last_stage = first_stage, last_stage
        lo, hi = layer_range if layer_range is not None else (0, args.n_layers)
        self.layer_range = (lo, hi)
        self.tp_group = ctx.tp_group if args.tp_size > 1 else None
        self.sp = args.sequence_parallel and args.tp_size > 1
        if first_stage:
            if args.tp_size > 1:
                self.tok_embeddings = VocabParallelEmbedding(args.vocab_size, args.dim, group=ctx.tp_group,
                                                             sequence_parallel=False, **kw)
            else:
                self.tok_embeddings = Embedding(args.vocab_size, args.dim, **kw)
        self.layers = nn.ModuleDict({str(i): TransformerBlock(args, i, ctx, **kw) for i in range(lo, hi)})
        if last_stage:
            self.norm = RMSNorm(args.dim, eps=args.norm_eps, **kw)
            if args.tp_size > 1:
                self.output = ColumnParallelLinear(args.dim, args.vocab_size, bias=False, gather_output=False,
                                                   group=ctx.tp_group, **kw)
            else:
                self.output = Linear(args.dim, args.vocab_size, **kw)
        self._rope_cache = None
        self.aux_losses: List[torch.Tensor] = []

    # ---- pieces -----------------------------------------------------------------------
    def rope_tables(self, device):
        c = self._rope_cache
        if c is None or c[0].device != device:
            cos, sin = ref.rope_tables(self.args.head_dim, self.args.max_seq_len, self.args.rope_theta, device=device)
            c = self._rope_cache = (cos.contiguous(), sin.contiguous())
        return c

    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, S] -> [T, H] (rows sharded over TP under sequence parallelism)."""
        flat = tokens.reshape(-1)
        if self.args.tp_size > 1:
            from ..parallel import embed_fused
            if embed_fused.fused_ok(self.tok_embeddings.weight, self.tp_group, flat.numel(), self.sp):
                # the owner of a token's id stores its row straight into the rank that needs it
                return embed_fused.vocab_parallel_embedding(flat, self.tok_embeddings.weight, self.tp_group,
                                                            self.tok_embeddings.vocab_start, self.sp)
            part = OF.embedding(flat, self.tok_embeddings.weight, self.tok_embeddings.vocab_start)
            if self.sp:
                return comm.scatter_rows(part, self.tp_group)
            return comm.reduce_from_group(part, self.tp_group)
        return OF.embedding(flat, self.tok_embeddings.weight, 0)

    def run_layers(self, h, delta, B, S, positions):
        cos, sin = self.rope_tables(h.device)
        if positions is not None and h.is_cuda:
            positions = positions.to(device=h.device, dtype=torch.int32)
        for blk in self.layers.values():
            h, delta = blk(h, delta, B, S, cos, sin, positions)
        return h, delta

    def head(self, h, delta) -> torch.Tensor:
        """Final norm + LM head -> local logits [T, V/tp] (rows gathered first under SP)."""
        if delta is None:
            x = OF.rmsnorm(h, self.norm.weight, self.norm.eps)
        else:
            _, x = OF.add_rmsnorm(delta, h, self.norm.weight, self.norm.eps)
        if self.sp:
            return fused.all_gather_linear(x, (self.output.weight,), self.tp_group)
        return OF.linear(comm.copy_to_group(x, self.tp_group), self.output.weight)

    # ---- stage-level API (pipeline parallel uses this directly) --------------------------
    def forward_stage(self, x: torch.Tensor, B: int, S: int, positions=None) -> torch.Tensor:
        """First stage: x = tokens [B,S]; other stages: x = hidden [T(/tp), H].
        Returns hidden [T(/tp), H], or local logits [T, V/tp] on the last stage."""
        self.aux_losses = []
        h = self.embed(x) if self.first_stage else x
        h, delta = self.run_layers(h, None, B, S, positions)
        if self.last_stage:
            return self.head(h, delta)
        return h if delta is None else h + delta

    def loss_from_logits(self, logits_local: torch.Tensor, targets: torch.Tensor,
                         n_tokens: Optional[int] = None) -> torch.Tensor:
        T = logits_local.shape[0]
        vs = comm.group_rank(self.tp_group) * logits_local.shape[-1]
        loss = OF.cross_entropy(logits_local, targets.reshape(-1), vs, self.tp_group, n_valid_total=n_tokens or T)
        return loss

    def collect_aux_loss(self):
        aux = None
        for blk in self.layers.values():
            a = getattr(blk.feed_forward, "last_aux_loss", None)
            if a is not None:
                aux = a if aux is None else aux + a
                blk.feed_forward.last_aux_loss = None
        return aux

    # ---- user-level API ---------------------------------------------------------------------
    def forward(self, tokens: torch.Tensor, positions=None) -> torch.Tensor:
        """tokens [B, S] -> logits [B, S, V] (full vocab on every TP rank, as the reference's
        ``gather_output=True`` head, model/model.py:243)."""
        assert self.first_stage and self.last_stage, "forward() needs the whole model; use forward_stage under PP"
        B, S = tokens.shape
        logits = self.forward_stage(tokens, B, S, positions)
        logits = comm.gather_cols(logits, self.tp_group)
        return logits.view(B, S, -1)

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor, positions=None,
             n_tokens: Optional[int] = None) -> torch.Tensor:
        """Token-mean next-token NLL (+ MoE aux loss) without materialising gathered logits."""
        B, S = tokens.shape
        logits = self.forward_stage(tokens, B, S, positions)
        loss = self.loss_from_logits(logits, targets, n_tokens)
        aux = self.collect_aux_loss()
        if aux is not None:
            loss = loss + self.args.moe_aux_loss_coef * aux
        return loss


# ---- parameter init and the flat arena ----------------------------------------------------------


def _full_shape(p: torch.Tensor, tp: int):
    shape = list(p.shape)
    dim = getattr(p, "tp_shard_dim", None)
    if dim is not None and tp > 1:
        shape[dim] *= tp
    return shape, dim


@torch.no_grad()
def init_weights(model: nn.Module, seed: int = 42, std: float = 0.02) -> None:
    """N(0, std) for every matrix, ones for norm weights (trainer.py:172-193 of the reference).
    Each parameter is drawn from a generator seeded by (seed, its name) at its FULL unsharded
    shape and then sliced, so the values do not depend on tp / pp / ep layout."""
    ctx = getattr(model, "ctx", None) or _mesh.get_context()
    tp, tpr = ctx.tp_size, ctx.tp_rank
    for name, p in model.named_parameters():
        if p.dim() == 1:
            p.fill_(1.0) if "norm" in name else p.zero_()
            continue
        shape, dim = _full_shape(p, tp)
        g = torch.Generator(device=p.device if p.is_cuda else "cpu")
        g.manual_seed((zlib.crc32(name.encode()) ^ (seed * 2654435761)) & 0x7FFFFFFF)
        full = torch.empty(shape, dtype=torch.float32, device=p.device).normal_(0.0, std, generator=g)
        if dim is not None and tp > 1:
            n = p.shape[dim]
            full = full.narrow(dim, tpr * n, n)
        p.copy_(full.to(p.dtype))


def flatten_parameters(model: nn.Module, dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Move every parameter into one contiguous arena (registration order, 256-byte aligned)
    and give every ``.grad`` a view into a second arena.  Row-adjacent q/k/v and gate/up
    weights then form single GEMM operands, zeroing grads is one memset, and the data-parallel
    reduce-scatter + AdamW kernel works on two flat buffers.  Returns (params, grads).
    ``optim.DistributedAdamW`` does this itself; call it directly only for optimizer-free use."""
    from ..optim import build_arena
    flat, grads, _, _ = build_arena(model, 1, 1, dtype)
    return flat, grads
