"""Checkpoint save / resume / re-shard.

The reference only saves, once, at the end, from global rank 0
(``torch.save({'model','optimizer','trained_steps','trained_tokens'}, './ckpt_step_{step}_tpsize_{tp}_dpsize_{dp}')``,
trainer.py:330-338), which under TP / FSDP / PP stores rank 0's shards only, and it has no load path.

Here the same dict keys and parameter names are kept, and:
* the ``model`` entry written by rank 0 is the FULL unsharded state_dict (TP shards concatenated,
  pipeline stages and expert shards merged), so the file loads into any parallel layout and into
  the reference's single-device model;
* every rank additionally writes ``<path>.opt/rank{r}.pt`` with its optimizer shard (fp32 master,
  moments), RNG state and data cursor for exact resume in the same layout;
* ``load`` re-shards the full model state for the current layout.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import mesh as _mesh
from .parallel import comm


def ckpt_name(step: int, tp: int, dp: int, save_dir: str = ".") -> str:
    return os.path.join(save_dir, f"ckpt_step_{step}_tpsize_{tp}_dpsize_{dp}")


def _shard_dim(name: str, p: torch.Tensor) -> Optional[int]:
    return getattr(p, "tp_shard_dim", None)


@torch.no_grad()
def full_state_dict(model: nn.Module, ctx: Optional[_mesh.ParallelContext] = None) -> Dict[str, torch.Tensor]:
    """Gather the unsharded state_dict on every rank of the model-parallel groups (CPU tensors).
    TP shards are concatenated along their shard dim; pipeline stages and expert shards are merged
    with ``all_gather_object``."""
    ctx = ctx or getattr(model, "ctx", None) or _mesh.get_context()
    stage = getattr(model, "stage", model)
    # sharded-parameter engines: a parameter's storage holds its values only while its block is gathered
    if getattr(stage, "_fsdp_native", None) is not None:
        out = stage._fsdp_native.full_state_dict()
        return _merge_over_groups(out, ctx)
    if getattr(stage, "_fsdp", None) is not None:
        return {k: v.cpu() for k, v in stage._fsdp.full_state_dict().items()}
    out: Dict[str, torch.Tensor] = {}
    for name, p in stage.named_parameters():
        t = p.detach()
        dim = _shard_dim(name, p)
        if dim is not None and ctx.tp_size > 1:
            parts = [torch.empty_like(t) for _ in range(ctx.tp_size)]
            dist.all_gather(parts, t.contiguous(), group=ctx.tp_group)
            t = torch.cat(parts, dim=dim)
        out[name] = t.cpu().clone()
    return _merge_over_groups(out, ctx)


def _merge_over_groups(out: Dict[str, torch.Tensor], ctx) -> Dict[str, torch.Tensor]:
    """Pipeline stages and expert-parallel ranks hold different parameters: union of their dicts."""
    for group, n in ((ctx.ep_group, ctx.ep_size), (ctx.pp_group, ctx.pp_size)):
        if n > 1:
            gathered = [None] * n
            dist.all_gather_object(gathered, out, group=group)
            merged: Dict[str, torch.Tensor] = {}
            for d in gathered:
                merged.update(d)
            out = merged
    return out


@torch.no_grad()
def load_full_state_dict(model: nn.Module, sd: Dict[str, torch.Tensor], ctx=None, strict: bool = True) -> None:
    """Copy a full (unsharded) state_dict into this rank's shards."""
    ctx = ctx or getattr(model, "ctx", None) or _mesh.get_context()
    stage = getattr(model, "stage", model)
    if getattr(stage, "_fsdp_native", None) is not None:
        return stage._fsdp_native.load_full_state_dict(sd)
    missing = []
    for name, p in stage.named_parameters():
        if name not in sd:
            missing.append(name)
            continue
        t = sd[name]
        dim = _shard_dim(name, p)
        if dim is not None and ctx.tp_size > 1:
            n = p.shape[dim]
            t = t.narrow(dim, ctx.tp_rank * n, n)
        if tuple(t.shape) != tuple(p.shape):
            raise ValueError(f"shape mismatch for {name}: checkpoint {tuple(t.shape)} vs model {tuple(p.shape)}")
        p.copy_(t.to(device=p.device, dtype=p.dtype))
    if strict and missing:
        raise KeyError(f"checkpoint is missing keys: {missing[:5]}{'...' if len(missing) > 5 else ''}")


def save(path: str, model: nn.Module, optimizer, step: int, tokens: int, dataloader=None, ctx=None,
         extra: Optional[Dict[str, Any]] = None) -> None:
    ctx = ctx or getattr(model, "ctx", None) or _mesh.get_context()
    full = full_state_dict(model, ctx)
    opt_dir = path + ".opt"
    if ctx.rank == 0:
        os.makedirs(opt_dir, exist_ok=True)
    if dist.is_initialized():
        dist.barrier()
    shard = {
        "optimizer": optimizer.state_dict() if optimizer is not None else None,
        "rng_cpu": torch.get_rng_state(),
        "rng_cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
        "data": dataloader.state_dict() if dataloader is not None else None,
        "layout": _layout_of(ctx),
    }
    tmp = os.path.join(opt_dir, f"rank{ctx.rank}.pt.tmp")
    torch.save(shard, tmp)
    os.replace(tmp, os.path.join(opt_dir, f"rank{ctx.rank}.pt"))
    if ctx.rank == 0:
        payload = {"model": full, "optimizer": {"sharded_in": os.path.basename(opt_dir)},
                   "trained_steps": step, "trained_tokens": tokens}
        if extra:
            payload.update(extra)
        torch.save(payload, path + ".tmp")
        os.replace(path + ".tmp", path)        # atomic: a crash never leaves a half-written file
    if dist.is_initialized():
        dist.barrier()


def _layout_of(ctx) -> Dict[str, int]:
    return {"tp": ctx.tp_size, "pp": ctx.pp_size, "cp": ctx.cp_size, "ep": ctx.ep_size, "dp": ctx.dp_size}


def _same_layout(shard: Dict[str, Any], optimizer, ctx) -> bool:
    """A rank's optimizer shard, RNG state and data cursor only mean something under the layout
    that wrote them (same tp / pp / cp / ep / dp sizes, hence the same shard of the same arena)."""
    saved = shard.get("layout")
    if saved is not None and {k: int(v) for k, v in saved.items()} != _layout_of(ctx):
        return False
    opt_sd = shard.get("optimizer")
    if opt_sd is not None and "shard_numel" in opt_sd and hasattr(optimizer, "shard_numel") \
            and opt_sd["shard_numel"] != optimizer.shard_numel:
        return False
    return True


def load(path: str, model: nn.Module, optimizer=None, dataloader=None, ctx=None) -> Dict[str, Any]:
    """Returns {'trained_steps', 'trained_tokens'}.  Raises on a corrupt / truncated file."""
    ctx = ctx or getattr(model, "ctx", None) or _mesh.get_context()
    try:
        payload = torch.load(path, map_location="cpu", weights_only=False)
    except Exception as e:
        raise RuntimeError(f"checkpoint {path} is unreadable (corrupt or truncated): {e}") from e
    for key in ("model", "trained_steps", "trained_tokens"):
        if key not in payload:
            raise RuntimeError(f"checkpoint {path} lacks '{key}'")
    load_full_state_dict(model, payload["model"], ctx)
    shard_file = os.path.join(path + ".opt", f"rank{ctx.rank}.pt")
    if optimizer is not None:
        shard = torch.load(shard_file, map_location="cpu", weights_only=False) if os.path.exists(shard_file) else None
        same_layout = shard is not None and _same_layout(shard, optimizer, ctx)
        if shard is not None and not same_layout:
            import warnings
            warnings.warn(f"checkpoint {path} was written with parallel layout {shard.get('layout')}, this run uses "
                          f"{_layout_of(ctx)}: weights are re-sharded; optimizer moments, RNG state and the data "
                          f"cursor of the old layout are not restored")
        if same_layout:
            if shard.get("optimizer") is not None:
                optimizer.load_state_dict(shard["optimizer"])
            if shard.get("rng_cpu") is not None:
                torch.set_rng_state(shard["rng_cpu"])
            if shard.get("rng_cuda") is not None and torch.cuda.is_available():
                torch.cuda.set_rng_state(shard["rng_cuda"])
            if dataloader is not None and shard.get("data") is not None:
                dataloader.load_state_dict(shard["data"])
        else:
            # different layout: weights are re-sharded, master weights restart from them, and the data
            # cursor is recomputed from the step count (one cursor tick per micro-batch of a rank)
            optimizer.refresh_master_from_params()
            if dataloader is not None and hasattr(dataloader, "cursor"):
                dataloader.cursor = int(payload["trained_steps"]) * int(getattr(dataloader, "grad_acc_steps", 1))
    return {"trained_steps": payload["trained_steps"], "trained_tokens": payload["trained_tokens"]}
