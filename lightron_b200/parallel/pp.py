"""Pipeline parallelism: stage construction, point-to-point exchange, AFAB and 1F1B schedules.

Parity with the reference: ``parallel/parallel_pp.py`` (even layer split ``:66-77``; first stage
owns the embedding, last stage owns norm + head ``:35-42``; manual stage backward ``:101-128``;
``train_step_pipeline_afab`` ``:131-183``; ``train_step_pipeline_1f1b`` with warm-up
``min(pp - rank - 1, n_mb)`` ``:186-293``) and ``parallel/communication/pipeline_parallel_p2p.py``
(``PPGroupManager`` ``:11-50``, uni- and bi-directional exchange ``:78-202``).

Differences: a stage builds only its own layers (the reference materialises the whole model on
every rank, trainer.py:218,246); PP composes with DP / TP / CP (the reference asserts dp == 1,
trainer.py:123-124) and gradient reduction is enabled only for the last micro-batch; the
exchange stays on NCCL send/recv as in the reference but never calls ``cuda.synchronize``
(pipeline_parallel_p2p.py:141,197): requests are waited on the stream, so the host keeps
running ahead and compute of other micro-batches overlaps the transfers; the loss is returned
as a device tensor (no ``.item()`` per micro-batch).
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import mesh as _mesh
from ..config import ModelArgs

VERBOSE = os.environ.get("VERBOSE", "0") == "1"


def distribute_layers(num_layers: int, pp_size: int, pp_rank: int) -> List[int]:
    per = [num_layers // pp_size + (1 if i < num_layers % pp_size else 0) for i in range(pp_size)]
    start = sum(per[:pp_rank])
    return list(range(start, start + per[pp_rank]))


class PPGroupManager:
    """Rank bookkeeping of one pipeline group (same attribute names as the reference)."""

    def __init__(self, ctx: Optional[_mesh.ParallelContext] = None):
        ctx = ctx or _mesh.get_context()
        self.ctx = ctx
        self.pp_group = ctx.pp_group
        self.pp_world_size = ctx.pp_size
        self.pp_rank = ctx.pp_rank
        self.pp_is_first_stage = ctx.pp_is_first
        self.pp_is_last_stage = ctx.pp_is_last
        self.pp_prev_rank = ctx.pp_prev_rank
        self.pp_next_rank = ctx.pp_next_rank
        self.global_rank = ctx.rank


_PPM: Optional[PPGroupManager] = None


def init_pp_group_manager(ctx=None) -> PPGroupManager:
    global _PPM
    _PPM = PPGroupManager(ctx)
    return _PPM


def get_pp_group_manager() -> PPGroupManager:
    return _PPM if _PPM is not None else init_pp_group_manager()


# ---- point-to-point -----------------------------------------------------------------------------

_STEP = 0


def _exchange(ppm: PPGroupManager, send_next=None, send_prev=None, recv_next_like=None, recv_prev_like=None):
    """Post every send / recv of this call as one batch, then wait on the stream.
    ``recv_*_like`` = (shape, dtype, device) or None.  Returns (from_prev, from_next)."""
    global _STEP
    ops, from_prev, from_next = [], None, None
    if recv_prev_like is not None:
        shape, dtype, device = recv_prev_like
        from_prev = torch.empty(shape, dtype=dtype, device=device)
        ops.append(dist.P2POp(dist.irecv, from_prev, ppm.pp_prev_rank))
    if send_next is not None:
        ops.append(dist.P2POp(dist.isend, send_next.contiguous(), ppm.pp_next_rank))
    if recv_next_like is not None:
        shape, dtype, device = recv_next_like
        from_next = torch.empty(shape, dtype=dtype, device=device)
        ops.append(dist.P2POp(dist.irecv, from_next, ppm.pp_next_rank))
    if send_prev is not None:
        ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), ppm.pp_prev_rank))
    if not ops:
        return None, None
    if VERBOSE:
        print(f"[pp p2p {_STEP}] rank {ppm.global_rank}: " + ", ".join(
            f"{'send' if o.op is dist.isend else 'recv'}->{o.peer}" for o in ops), flush=True)
    _STEP += 1
    for req in dist.batch_isend_irecv(ops):
        req.wait()
    return from_prev, from_next


def pipeline_communicate(operation: str, device, dtype, tensor=None, shapes=None, ppm=None):
    """Uni-directional exchange, by the reference's operation names."""
    ppm = ppm or get_pp_group_manager()
    like = (shapes, dtype, device)
    if operation == "recv_forward":
        if ppm.pp_is_first_stage:
            return None
        t, _ = _exchange(ppm, recv_prev_like=like)
        return t.requires_grad_(True)
    if operation == "send_forward":
        if not ppm.pp_is_last_stage:
            _exchange(ppm, send_next=tensor)
        return None
    if operation == "recv_backward":
        if ppm.pp_is_last_stage:
            return None
        _, t = _exchange(ppm, recv_next_like=like)
        return t
    if operation == "send_backward":
        if not ppm.pp_is_first_stage:
            _exchange(ppm, send_prev=tensor)
        return None
    raise ValueError(f"unknown pipeline operation {operation}")


def bidirectional_pipeline_communicate(operation: str, send_tensor, recv_shapes, device, dtype, ppm=None):
    ppm = ppm or get_pp_group_manager()
    like = (recv_shapes, dtype, device)
    if operation == "send_fwd_recv_bwd":
        if ppm.pp_is_last_stage:
            return None
        _, t = _exchange(ppm, send_next=send_tensor, recv_next_like=like)
        return t
    if operation == "send_bwd_recv_fwd":
        if ppm.pp_is_first_stage:
            return None
        t, _ = _exchange(ppm, send_prev=send_tensor, recv_prev_like=like)
        return t.requires_grad_(True)
    raise ValueError(f"unknown pipeline operation {operation}")


# ---- stage --------------------------------------------------------------------------------------


class PipelineParallel(nn.Module):
    """One pipeline stage.  ``PipelineParallel(model_args)`` builds just this stage's layers;
    ``PipelineParallel(full_model, model_args)`` (the reference's calling convention) keeps the
    stage's modules of an already built model."""

    def __init__(self, model_or_args, model_args: Optional[ModelArgs] = None, ctx=None, dtype=None, device=None):
        super().__init__()
        from ..models.llama import LightronTransformer
        self.ppm = PPGroupManager(ctx)
        ctx = self.ppm.ctx
        if isinstance(model_or_args, ModelArgs):
            args = model_or_args
            ids = distribute_layers(args.n_layers, ctx.pp_size, ctx.pp_rank)
            self.stage = LightronTransformer(args, ctx, layer_range=(ids[0], ids[-1] + 1),
                                             first_stage=ctx.pp_is_first, last_stage=ctx.pp_is_last,
                                             dtype=dtype, device=device)
        else:
            full, args = model_or_args, model_args
            ids = distribute_layers(args.n_layers, ctx.pp_size, ctx.pp_rank)
            keep = {str(i) for i in ids}
            for k in list(full.layers.keys()):
                if k not in keep:
                    del full.layers[k]
            if not ctx.pp_is_first and hasattr(full, "tok_embeddings"):
                del full.tok_embeddings
            if not ctx.pp_is_last:
                for nme in ("norm", "output"):
                    if hasattr(full, nme):
                        delattr(full, nme)
            full.first_stage, full.last_stage = ctx.pp_is_first, ctx.pp_is_last
            full.layer_range = (ids[0], ids[-1] + 1)
            self.stage = full
        self.model_args = args
        self.ctx = ctx
        self.args = args
        self.layer_distribution = ids

    # state_dict keys carry no wrapper prefix: global layer indices, plain names.
    def state_dict(self, *a, **kw):
        return self.stage.state_dict(*a, **kw)

    def load_state_dict(self, sd, *a, **kw):
        return self.stage.load_state_dict(sd, *a, **kw)

    def forward(self, input_ids=None, hidden_states=None, B=None, S=None, positions=None):
        x = hidden_states if hidden_states is not None else input_ids
        return self.stage.forward_stage(x, B, S, positions)

    def backward(self, input_tensor, output_tensor, output_tensor_grad):
        if input_tensor is not None:
            input_tensor.retain_grad()
        if output_tensor_grad is None:
            output_tensor_grad = torch.ones_like(output_tensor)
        torch.autograd.backward(output_tensor, grad_tensors=output_tensor_grad)
        return input_tensor.grad if input_tensor is not None else None


# ---- schedules ------------------------------------------------------------------------------------


def _set_sync(optimizer, flag: bool):
    if optimizer is not None and hasattr(optimizer, "set_requires_gradient_sync"):
        optimizer.set_requires_gradient_sync(flag)


class _Stepper:
    """Shared forward / backward micro-step logic of both schedules."""

    def __init__(self, model: PipelineParallel, data_iter, tensor_shapes, device, dtype, positions=None):
        self.model, self.data_iter = model, data_iter
        self.shapes, self.device, self.dtype = tuple(tensor_shapes), device, dtype
        self.ppm = model.ppm
        self.n_mb = data_iter.grad_acc_steps
        self.positions = positions
        self.loss_sum = torch.zeros((), dtype=torch.float32, device=device)

    def forward_step(self, input_tensor):
        batch = next(self.data_iter)              # every stage draws the batch: same cursor everywhere
        B, S = batch["input_ids"].shape
        if self.ppm.pp_is_first_stage:
            out = self.model(input_ids=batch["input_ids"].to(self.device, non_blocking=True), B=B, S=S,
                             positions=self.positions)
        else:
            out = self.model(hidden_states=input_tensor, B=B, S=S, positions=self.positions)
        if self.ppm.pp_is_last_stage:
            tgt = batch["target_ids"].to(self.device, non_blocking=True)
            loss = self.model.stage.loss_from_logits(out, tgt)
            aux = self.model.stage.collect_aux_loss()
            if aux is not None:
                loss = loss + self.model.args.moe_aux_loss_coef * aux
            out = loss / self.n_mb
            self.loss_sum += out.detach().float()
        return out


def train_step_pipeline_afab(model: PipelineParallel, data_iter, tensor_shapes, device, dtype, optimizer=None,
                             positions=None) -> torch.Tensor:
    """All-forward-all-backward.  Returns the summed micro-batch loss (a device scalar; zero on
    stages other than the last)."""
    st = _Stepper(model, data_iter, tensor_shapes, device, dtype, positions)
    ppm = st.ppm
    ins, outs = [], []
    _set_sync(optimizer, False)
    for _ in range(st.n_mb):
        x = pipeline_communicate("recv_forward", device, dtype, shapes=st.shapes, ppm=ppm)
        y = st.forward_step(x)
        pipeline_communicate("send_forward", device, dtype, tensor=y.detach() if not ppm.pp_is_last_stage else None, ppm=ppm)
        ins.append(x)
        outs.append(y)
    for i in range(st.n_mb):
        _set_sync(optimizer, i == st.n_mb - 1)
        g = pipeline_communicate("recv_backward", device, dtype, shapes=st.shapes, ppm=ppm)
        x, y = ins.pop(0), outs.pop(0)
        gx = model.backward(x, y, g)
        pipeline_communicate("send_backward", device, dtype, tensor=gx, ppm=ppm)
    return st.loss_sum


def train_step_pipeline_1f1b(model: PipelineParallel, data_iter, tensor_shapes, device, dtype, optimizer=None,
                             positions=None) -> torch.Tensor:
    """One-forward-one-backward: warm-up forwards, steady 1F1B pairs, cool-down backwards."""
    st = _Stepper(model, data_iter, tensor_shapes, device, dtype, positions)
    ppm = st.ppm
    n_warm = min(ppm.pp_world_size - ppm.pp_rank - 1, st.n_mb)
    n_rem = st.n_mb - n_warm
    ins, outs = [], []
    _set_sync(optimizer, False)

    def detached(y):
        return None if ppm.pp_is_last_stage else y.detach()

    for _ in range(n_warm):
        x = pipeline_communicate("recv_forward", device, dtype, shapes=st.shapes, ppm=ppm)
        y = st.forward_step(x)
        pipeline_communicate("send_forward", device, dtype, tensor=detached(y), ppm=ppm)
        ins.append(x)
        outs.append(y)
    x = pipeline_communicate("recv_forward", device, dtype, shapes=st.shapes, ppm=ppm) if n_rem > 0 else None
    for i in range(n_rem):
        last = i == n_rem - 1
        y = st.forward_step(x)
        g = bidirectional_pipeline_communicate("send_fwd_recv_bwd", detached(y), st.shapes, device, dtype, ppm=ppm)
        ins.append(x)
        outs.append(y)
        xi, yi = ins.pop(0), outs.pop(0)
        if n_warm == 0 and last:
            _set_sync(optimizer, True)
        gx = model.backward(xi, yi, g)
        if last:
            x = None
            pipeline_communicate("send_backward", device, dtype, tensor=gx, ppm=ppm)
        else:
            x = bidirectional_pipeline_communicate("send_bwd_recv_fwd", gx, st.shapes, device, dtype, ppm=ppm)
    for i in range(n_warm):
        if i == n_warm - 1:
            _set_sync(optimizer, True)
        g = pipeline_communicate("recv_backward", device, dtype, shapes=st.shapes, ppm=ppm)
        xi, yi = ins.pop(0), outs.pop(0)
        gx = model.backward(xi, yi, g)
        pipeline_communicate("send_backward", device, dtype, tensor=gx, ppm=ppm)
    return st.loss_sum
