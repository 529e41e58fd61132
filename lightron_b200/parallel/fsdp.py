"""Fully sharded data parallelism (parameters, gradients and optimizer state sharded over DP).

API parity with the reference's ``parallel/parallel_fsdp.py``: ``apply_fsdp2`` (``:115-183``:
``fully_shard`` per transformer block, then the root, bf16 parameters, fp32 gradient reduction,
``reshard_after_forward``) and ``apply_fsdp1`` (``:38-112``: FULL_SHARD / SHARD_GRAD_OP / HYBRID
strategies, optional activation checkpointing).  The reference delegates to PyTorch's FSDP; this
is a small self-contained implementation so that the unit of sharding, the collectives and the
dtype policy are ours:

* every block owns ONE flat fp32 master shard (1/n of its parameters, a real ``nn.Parameter``
  that the optimizer steps) and one flat compute buffer in the parameter dtype whose storage is
  released between uses (``storage.resize_(0)``), so tensors that autograd saved as views of it
  see the re-gathered values in backward;
* unshard = one all-gather of the block's flat buffer before its forward and before its
  backward; reshard after forward (FULL_SHARD) or keep (SHARD_GRAD_OP);
* after the block's last parameter gradient has been accumulated, the flat gradient is
  reduce-scattered in ``reduce_dtype`` (fp32 by default) into the master shard's ``.grad``;
  with ``set_requires_gradient_sync(False)`` gradients accumulate locally (the reference
  reduces on every micro-batch).

The trainer's default data-parallel engine is ``optim.DistributedAdamW`` (replicated bf16
parameters, sharded optimizer state), which needs no per-block all-gathers at all on a 180 GB
GPU; this module is the choice when parameters themselves must be sharded.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import mesh as _mesh
from . import comm

_ALIGN = 128


class _ShardedUnit:
    def __init__(self, name: str, params: List[nn.Parameter], names: List[str], group, param_dtype, reduce_dtype,
                 reshard_after_forward: bool, keep_resident: bool = False):
        self.name, self.params, self.names, self.group = name, params, names, group
        self.keep_resident = keep_resident      # root unit: used outside module calls, never freed
        self.n, self.rank = comm.group_size(group), comm.group_rank(group)
        self.param_dtype, self.reduce_dtype = param_dtype, reduce_dtype
        self.reshard_after_forward = reshard_after_forward
        self.shapes = [p.shape for p in params]
        self.offsets, total = [], 0
        for p in params:
            self.offsets.append(total)
            total += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        unit = _ALIGN * self.n
        self.total = (total + unit - 1) // unit * unit
        self.shard_len = self.total // self.n
        device = params[0].device
        full = torch.zeros(self.total, dtype=torch.float32, device=device)
        for p, off in zip(params, self.offsets):
            full[off:off + p.numel()].copy_(p.data.reshape(-1).float())
        self.shard = nn.Parameter(full[self.rank * self.shard_len:(self.rank + 1) * self.shard_len].clone())
        self.full = torch.empty(self.total, dtype=param_dtype, device=device)
        self.nbytes = self.full.untyped_storage().size()
        self.sharded = False
        self.sync = True
        self.pending = 0
        for p, off, shape in zip(params, self.offsets, self.shapes):
            p.data = self.full[off:off + p.numel()].view(shape)
            p.register_post_accumulate_grad_hook(self._grad_hook)
        self.unshard(force=True)
        self.reshard()

    # ---- parameter lifetime ------------------------------------------------------------------
    def unshard(self, force: bool = False) -> None:
        if not self.sharded and not force:
            return
        st = self.full.untyped_storage()
        if st.size() != self.nbytes:
            st.resize_(self.nbytes)
        local = self.shard.detach().to(self.param_dtype)
        if self.n == 1:
            self.full.copy_(local)
        else:
            dist.all_gather_into_tensor(self.full, local, group=self.group)
        self.sharded = False

    def reshard(self) -> None:
        if self.n == 1 or self.keep_resident:
            return
        self.full.untyped_storage().resize_(0)
        self.sharded = True

    # ---- gradients -----------------------------------------------------------------------------
    def _grad_hook(self, _p) -> None:
        if self.pending <= 0:                   # first gradient of a new backward pass
            self.pending = sum(1 for p in self.params if p.requires_grad)
        self.pending -= 1
        if self.pending == 0:
            self.post_backward()

    def pre_backward(self) -> None:
        self.unshard()

    def post_backward(self) -> None:
        if not self.sync:
            self.unsynced = True
            return
        flat = torch.zeros(self.total, dtype=self.reduce_dtype, device=self.shard.device)
        for p, off in zip(self.params, self.offsets):
            if p.grad is not None:
                flat[off:off + p.numel()].copy_(p.grad.reshape(-1))
                p.grad = None
        if self.n > 1:
            g = comm.reduce_scatter_rows(flat.view(self.n, self.shard_len), self.group).view(-1) / self.n
        else:
            g = flat
        g = g.to(self.shard.dtype)
        self.shard.grad = g if self.shard.grad is None else self.shard.grad + g
        self.reshard()

    @torch.no_grad()
    def full_tensors(self) -> Dict[str, torch.Tensor]:
        was = self.sharded
        self.unshard()
        out = {n: self.full[off:off + int(torch.Size(s).numel())].view(s).detach().clone()
               for n, off, s in zip(self.names, self.offsets, self.shapes)}
        if was:
            self.reshard()
        return out


class FSDPState:
    """Attached to the wrapped model as ``model._fsdp``."""

    def __init__(self):
        self.units: List[_ShardedUnit] = []

    def parameters(self) -> Iterable[nn.Parameter]:
        return [u.shard for u in self.units]

    def set_requires_gradient_sync(self, flag: bool) -> None:
        for u in self.units:
            u.sync = bool(flag)

    def refresh(self) -> None:
        """Re-gather the units that stay resident (call after every optimizer step; the optimizer
        returned by ``make_optimizer`` does it by itself)."""
        for u in self.units:
            if u.keep_resident:
                u.unshard(force=True)

    def make_optimizer(self, lr: float = 3e-4, weight_decay: float = 0.01, betas=(0.9, 0.999), eps: float = 1e-8):
        opt = torch.optim.AdamW(self.parameters(), lr=lr, weight_decay=weight_decay, betas=betas, eps=eps)
        opt.register_step_post_hook(lambda *_a, **_k: self.refresh())
        return opt

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for u in self.units:
            out.update(u.full_tensors())
        return out


def _wrap(module: nn.Module, unit: _ShardedUnit, checkpoint: bool) -> None:
    def pre_fwd(_m, _inp):
        unit.unshard()

    def post_fwd(_m, _inp, out):
        if unit.reshard_after_forward and torch.is_grad_enabled():
            # backward re-gathers; tensors saved for backward are views of the same storage
            unit.reshard()
        return out

    def pre_bwd(_m, _gout):
        unit.pre_backward()

    module.register_forward_pre_hook(pre_fwd)
    module.register_forward_hook(post_fwd)
    module.register_full_backward_pre_hook(pre_bwd)
    if checkpoint:
        from torch.utils.checkpoint import checkpoint as ckpt
        inner = module.forward
        module.forward = lambda *a, **kw: ckpt(inner, *a, use_reentrant=False, **kw)


def apply_fsdp2(model: nn.Module, ctx: Optional[_mesh.ParallelContext] = None, param_dtype: Optional[torch.dtype] = None,
                reduce_dtype: torch.dtype = torch.float32, reshard_after_forward: bool = True,
                activation_checkpointing: bool = False) -> nn.Module:
    """Shard every transformer block, then the remaining (root) parameters, over the DP group.
    Optimise ``model._fsdp.parameters()`` (fp32 master shards)."""
    ctx = ctx or getattr(model, "ctx", None) or _mesh.get_context()
    group = ctx.dp_group
    state = FSDPState()
    seen = set()
    param_dtype = param_dtype or next(model.parameters()).dtype
    blocks = list(model.layers.values()) if hasattr(model, "layers") and hasattr(model.layers, "values") else \
        (list(model.layers) if hasattr(model, "layers") else [])
    prefix_of = {id(m): n for n, m in model.named_modules()}
    for blk in blocks:
        named = [(f"{prefix_of[id(blk)]}.{n}", p) for n, p in blk.named_parameters()]
        unit = _ShardedUnit(prefix_of[id(blk)], [p for _, p in named], [n for n, _ in named], group, param_dtype,
                            reduce_dtype, reshard_after_forward)
        seen.update(id(p) for _, p in named)
        _wrap(blk, unit, activation_checkpointing)
        state.units.append(unit)
    rest = [(n, p) for n, p in model.named_parameters() if id(p) not in seen]
    if rest:
        unit = _ShardedUnit("root", [p for _, p in rest], [n for n, _ in rest], group, param_dtype, reduce_dtype,
                            reshard_after_forward=False, keep_resident=True)   # embedding / head / final norm
        unit.unshard(force=True)
        state.units.append(unit)
    model._fsdp = state
    return model


def apply_fsdp1(model: nn.Module, strategy: str = "full", activation_checkpointing: bool = False,
                ctx: Optional[_mesh.ParallelContext] = None, param_dtype: Optional[torch.dtype] = None) -> nn.Module:
    """FULL_SHARD ("full"), SHARD_GRAD_OP ("grad_op": parameters stay gathered between forward and
    backward) or HYBRID ("hybrid": shard inside the node, replicate across nodes; on one NVSwitch
    box this is FULL_SHARD)."""
    if strategy not in ("full", "grad_op", "hybrid"):
        raise ValueError(f"unknown FSDP strategy {strategy}")
    return apply_fsdp2(model, ctx=ctx, param_dtype=param_dtype, reshard_after_forward=(strategy != "grad_op"),
                       activation_checkpointing=activation_checkpointing)


class FSDPOptimizer:
    """The trainer-facing optimizer of a model wrapped by :func:`apply_fsdp2` (library collectives,
    ``torch.optim.AdamW`` on the fp32 master shards): the same small interface as
    ``optim.DistributedAdamW`` and ``fsdp_native.NativeFSDP``."""

    def __init__(self, model: nn.Module, lr: float, weight_decay: float, betas=(0.9, 0.999), eps: float = 1e-8):
        self.model, self.state = model, model._fsdp
        self.opt = self.state.make_optimizer(lr=lr, weight_decay=weight_decay, betas=betas, eps=eps)
        self.step_count = 0
        self.shard_numel = sum(u.shard_len for u in self.state.units)

    def set_requires_gradient_sync(self, flag: bool) -> None:
        self.state.set_requires_gradient_sync(flag)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.opt.zero_grad(set_to_none=True)

    def finish_grad_sync(self) -> None:
        pass

    def step(self) -> None:
        self.opt.step()
        self.step_count += 1

    def refresh_master_from_params(self) -> None:
        pass

    def state_dict(self):
        return {"step": self.step_count, "torch": self.opt.state_dict(), "shard_numel": self.shard_numel,
                "masters": [u.shard.detach().cpu() for u in self.state.units]}

    def load_state_dict(self, sd) -> None:
        assert sd["shard_numel"] == self.shard_numel, "optimizer shard layout differs"
        self.step_count = int(sd["step"])
        with torch.no_grad():
            for u, m in zip(self.state.units, sd["masters"]):
                u.shard.copy_(m)
        self.opt.load_state_dict(sd["torch"])
        self.state.refresh()
