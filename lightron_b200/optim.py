"""Sharded AdamW over the flat parameter / gradient arenas.

Replaces three reference pieces at once: ``torch.optim.AdamW`` on bf16 parameters
(trainer.py:268-272,315: no fp32 master copy, Adam moments in bf16), the per-parameter DDP
all-reduce hook (parallel/parallel_dp.py:27-38: one collective per tensor per micro-batch) and the
FSDP2 gradient reduce-scatter that fires on every micro-batch (parallel/parallel_fsdp.py:167-181).

Design: gradients live in one flat arena cut into buckets.  When the last gradient of a bucket
has been accumulated (autograd post-accumulate hooks) and gradient sync is enabled (last
micro-batch only), the bucket is reduce-scattered over the replica group (dp x cp) on a side
stream while backward continues.  Each rank owns 1/n of every bucket: fp32 master weights and
Adam moments exist only for that shard (ZeRO-1/2), the fused AdamW kernel reads the reduced bf16
gradient shard and writes both the fp32 master and the bf16 parameter shard, and one all-gather per
bucket refreshes the replicated bf16 parameters.  With 180 GB per GPU the bf16 parameters stay
replicated, which removes FSDP2's per-block all-gathers from the forward and backward passes.
Expert parameters use their own replica group (dp/ep x cp).
"""
from __future__ import annotations

import math
import os
import ctypes
from contextlib import contextmanager
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import mesh as _mesh
from .ops import functional as OF, native, reference as ref
from .parallel import comm

_ALIGN = 128


class _Bucket:
    __slots__ = ("start", "end", "group", "n", "shard_len", "shard_off", "pending", "n_params", "launched", "event", "seen",
                 "post_scale")

    def __init__(self, start, end, group, n, shard_off, post_scale=1.0):
        self.start, self.end, self.group, self.n = start, end, group, n
        self.post_scale = post_scale
        self.shard_len = (end - start) // n
        self.shard_off = shard_off
        self.pending = self.n_params = 0
        self.launched = False
        self.event = None
        self.seen = set()


def arrange_parameters(model: nn.Module) -> List[nn.Parameter]:
    """Arena order: dense parameters in registration order, then expert parameters (which are
    reduced over a different replica group and therefore need their own contiguous region)."""
    dense = [p for p in model.parameters() if not getattr(p, "is_expert", False)]
    expert = [p for p in model.parameters() if getattr(p, "is_expert", False)]
    return dense + expert


@torch.no_grad()
def build_arena(model: nn.Module, n_dense: int, n_expert: int, dtype: Optional[torch.dtype] = None, allocator=None):
    """Lay parameters out in a flat arena: [dense region | expert region], every region padded
    so that it splits evenly (and 128-element aligned) over its replica group.
    ``allocator(total_elements, dtype, device) -> (params, grads)`` lets the caller place both
    arenas in peer-visible (symmetric) memory."""
    params = arrange_parameters(model)
    dtype = dtype or params[0].dtype
    device = params[0].device
    offs, total = [], 0
    dense_end = 0
    for p in params:
        if getattr(p, "is_expert", False) and dense_end == 0 and total > 0:
            pad = _ALIGN * n_dense
            total = (total + pad - 1) // pad * pad
            dense_end = total
        offs.append(total)
        total += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
    has_expert = any(getattr(p, "is_expert", False) for p in params)
    if not has_expert:
        pad = _ALIGN * n_dense
        total = (total + pad - 1) // pad * pad
        dense_end = total
    else:
        pad = _ALIGN * n_expert
        total = (total + pad - 1) // pad * pad
    if allocator is not None:
        flat, grads = allocator(total, dtype, device)
    else:
        flat = torch.zeros(total, dtype=dtype, device=device)
        grads = torch.zeros(total, dtype=dtype, device=device)
    for p, off in zip(params, offs):
        view = flat[off:off + p.numel()].view(p.shape)
        view.copy_(p.data.to(dtype))
        p.data = view
        p.grad = grads[off:off + p.numel()].view(p.shape)
        p._arena_offset = off
    model._flat_params, model._flat_grads, model._arena_dense_end = flat, grads, dense_end
    return flat, grads, dense_end, offs


class DistributedAdamW:
    def __init__(self, model: nn.Module, lr: float = 3e-4, weight_decay: float = 0.01, betas=(0.9, 0.999),
                 eps: float = 1e-8, ctx: Optional[_mesh.ParallelContext] = None, bucket_mb: float = 256.0,
                 overlap: bool = True, grad_clip: float = 0.0, param_dtype: Optional[torch.dtype] = None):
        self.model = model
        self.ctx = ctx or getattr(model, "ctx", None) or _mesh.get_context()
        self.lr, self.weight_decay, self.betas, self.eps = lr, weight_decay, tuple(betas), eps
        self.grad_clip = grad_clip
        self.step_count = 0
        ctx = self.ctx
        n_dense = comm.group_size(ctx.dpcp_group)
        n_expert = comm.group_size(ctx.edpcp_group)
        # One kernel for reduce-scatter + AdamW + all-gather over NVLink peer memory when the
        # replica group allows it (arenas then live in symmetric memory).
        self.fused_dp = None
        allocator = None
        first = next(model.parameters())
        want_dtype = param_dtype or first.dtype
        has_expert = any(getattr(p, "is_expert", False) for p in model.parameters())
        if (first.is_cuda and want_dtype == torch.bfloat16 and n_dense > 1 and n_dense <= 8 and not has_expert
                and grad_clip <= 0 and native.available() and os.environ.get("LIGHTRON_FUSED_DP", "1") != "0"
                and dist.get_backend(ctx.dpcp_group) == "nccl"):
            allocator = self._symmetric_allocator
            bucket_mb = float("inf")          # a single shard range: one launch per step
        flat, grads, dense_end, offs = build_arena(model, n_dense, n_expert, param_dtype, allocator)
        self.flat_params, self.flat_grads = flat, grads
        self.params = arrange_parameters(model)
        self.device = flat.device
        self.native = flat.is_cuda and flat.dtype == torch.bfloat16 and native.available()
        if flat.is_cuda and flat.dtype == torch.bfloat16:
            native.require()
        # ---- buckets ----
        self.buckets: List[_Bucket] = []
        shard_off = 0
        # An expert's autograd gradient already holds the sum over the ep source ranks whose tokens it
        # served (the all-to-all backward brings them in), while the replica-group average below only
        # divides by the dp/ep x cp replicas: 1/ep_size completes the mean over all data-parallel ranks.
        ep_scale = 1.0 / max(1, int(getattr(ctx, "ep_size", 1)))
        for (lo, hi, group, n, post) in ((0, dense_end, ctx.dpcp_group, n_dense, 1.0),
                                         (dense_end, flat.numel(), ctx.edpcp_group, n_expert, ep_scale)):
            if hi <= lo:
                continue
            unit = _ALIGN * n
            target = hi - lo if bucket_mb == float("inf") else \
                max(unit, int(bucket_mb * (1 << 20) / flat.element_size()) // unit * unit)
            s = lo
            while s < hi:
                e = min(hi, s + target)
                b = _Bucket(s, e, group, n, shard_off, post)
                shard_off += b.shard_len
                self.buckets.append(b)
                s = e
        self.shard_numel = shard_off
        # ---- shard state: fp32 master / moments; gradient and parameter shard staging ----
        self.master = torch.empty(shard_off, dtype=torch.float32, device=self.device)
        for b in self.buckets:
            r = comm.group_rank(b.group)
            src = flat[b.start + r * b.shard_len: b.start + (r + 1) * b.shard_len]
            self.master[b.shard_off:b.shard_off + b.shard_len].copy_(src.float())
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        if all(b.n == 1 and b.shard_off == b.start for b in self.buckets) and shard_off == flat.numel():
            # no replicas: the "shards" are the arenas themselves (saves two full-arena copies per step)
            self.grad_shard, self.param_shard = self.flat_grads, self.flat_params
        else:
            self.grad_shard = torch.zeros(shard_off, dtype=flat.dtype, device=self.device)
            self.param_shard = torch.empty(shard_off, dtype=flat.dtype, device=self.device)
        # ---- hooks for overlapped reduction ----
        self.sync_enabled = True
        self.overlap = overlap and flat.is_cuda and any(b.n > 1 for b in self.buckets) and self.fused_dp is None
        self.comm_stream = torch.cuda.Stream() if self.overlap else None
        for p, off in zip(self.params, offs):
            for b in self.buckets:          # a tensor that straddles a bucket boundary counts in both
                if off < b.end and off + p.numel() > b.start:
                    b.n_params += 1
                    if self.overlap and p.requires_grad:
                        hook = self._make_hook(b)
                        p.register_post_accumulate_grad_hook(hook)
                        # ops that write a gradient straight into the arena (no autograd
                        # accumulation, hence no post-accumulate callback) call these themselves
                        p._lb_grad_hooks = getattr(p, "_lb_grad_hooks", ()) + (hook,)
            p._lb_direct_grad = bool(flat.is_cuda and flat.dtype == torch.bfloat16 and native.available())
        self._reset_buckets()
        # parameters whose gradient is a partial sum over the TP group (norm weights under
        # sequence parallelism: every TP rank saw only its own rows)
        self.sp_partial = [p for n_, p in model.named_parameters()
                           if getattr(getattr(model, "args", None), "sequence_parallel", False)
                           and ctx.tp_size > 1 and p.dim() == 1]

    # ---- peer-memory arenas for the fused reduce-scatter + AdamW + all-gather kernel -----------
    def _symmetric_allocator(self, total: int, dtype, device):
        import torch.distributed._symmetric_memory as symm_mem
        group = self.ctx.dpcp_group
        head = 4096                                       # flag words live in front of the arenas
        nbytes = head + 2 * total * 2
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        buf.zero_()
        hdl = symm_mem.rendezvous(buf, group=group)
        torch.cuda.synchronize()
        dist.barrier(group=group)
        ptrs = [int(x) + int(getattr(hdl, 'offset', 0)) for x in hdl.buffer_ptrs]
        n = dist.get_world_size(group)
        mk = lambda off: (ctypes.c_void_p * n)(*[p + off for p in ptrs])
        flat = buf[head:head + total * 2].view(dtype)
        grads = buf[head + total * 2:head + 4 * total].view(dtype)
        self.fused_dp = {"buf": buf, "hdl": hdl, "flags": mk(0), "params": mk(head), "grads": mk(head + total * 2),
                         "counter": torch.zeros(1, dtype=torch.int32, device=device), "epoch": 0,
                         "rank": dist.get_rank(group), "n": n, "grid": native.sm_count() * 8}
        return flat, grads

    # ---- gradient synchronisation ---------------------------------------------------------
    def _reset_buckets(self):
        for b in self.buckets:
            b.pending, b.launched, b.event, b.seen = b.n_params, False, None, set()

    def _make_hook(self, b: _Bucket):
        def hook(p):
            # Counts every parameter once per synchronised backward pass.  An op that wrote the
            # gradient straight into the arena calls this by hand, and autograd may call it again
            # for the same parameter (it runs the post-accumulate callbacks even when the op
            # returned no gradient), hence the set.  Micro-batches without sync do not count.
            if not self.sync_enabled or id(p) in b.seen or getattr(p, "_lb_wgrad_pending", False):
                return                      # (a queued weight gradient calls back when it has been launched)
            b.seen.add(id(p))
            b.pending -= 1
            if b.pending == 0 and not self.sp_partial:
                self._launch_reduce(b, async_op=True)
        return hook

    def _launch_reduce(self, b: _Bucket, async_op: bool):
        if b.launched:
            return
        b.launched = True
        g = self.flat_grads[b.start:b.end]
        out = self.grad_shard[b.shard_off:b.shard_off + b.shard_len]
        if b.n == 1:
            if out.data_ptr() != g.data_ptr():
                out.copy_(g)
            if b.post_scale != 1.0:
                out.mul_(b.post_scale)
            return
        if async_op and self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self._reduce_scatter(g, out, b)
                if b.post_scale != 1.0:
                    out.mul_(b.post_scale)
                b.event = torch.cuda.Event()
                b.event.record(self.comm_stream)
        else:
            self._reduce_scatter(g, out, b)
            if b.post_scale != 1.0:
                out.mul_(b.post_scale)

    def _reduce_scatter(self, g, out, b: _Bucket):
        if dist.get_backend(b.group) == "gloo":
            tmp = g.clone()
            dist.all_reduce(tmp, group=b.group)
            r = dist.get_rank(b.group)
            out.copy_(tmp[r * b.shard_len:(r + 1) * b.shard_len] / b.n)
        else:
            dist.reduce_scatter_tensor(out, g, op=dist.ReduceOp.AVG, group=b.group)

    @contextmanager
    def no_sync(self):
        """Skip gradient reduction (all micro-batches but the last)."""
        old = self.sync_enabled
        self.sync_enabled = False
        try:
            yield
        finally:
            self.sync_enabled = old

    def set_requires_gradient_sync(self, flag: bool) -> None:
        self.sync_enabled = bool(flag)

    def finish_grad_sync(self):
        OF.flush_wgrads()                   # normally empty: the queue is flushed when backward ends
        if self.sp_partial:
            buf = torch.cat([p.grad.reshape(-1).float() for p in self.sp_partial])
            dist.all_reduce(buf, group=self.ctx.tp_group)
            off = 0
            for p in self.sp_partial:
                p.grad.copy_(buf[off:off + p.numel()].view_as(p.grad))
                off += p.numel()
        if self.fused_dp is not None:
            return
        for b in self.buckets:
            self._launch_reduce(b, async_op=False)
        for b in self.buckets:
            if b.event is not None:
                torch.cuda.current_stream().wait_event(b.event)

    # ---- step -----------------------------------------------------------------------------
    def _clip_scale(self) -> float:
        if self.grad_clip <= 0:
            return 1.0
        sq = self.grad_shard.float().pow(2).sum()
        # every shard holds distinct elements of this rank's parameters; sum over the replica
        # group, then over TP / PP (different parameters).  Replicated tensors inside a TP group
        # are counted tp times, which only makes clipping marginally more conservative.
        for g in (self.ctx.dpcp_group, self.ctx.tp_group, self.ctx.pp_group):
            if comm.group_size(g) > 1:
                dist.all_reduce(sq, group=g)
        norm = math.sqrt(float(sq))
        self.last_grad_norm = norm
        return min(1.0, self.grad_clip / (norm + 1e-6))

    @torch.no_grad()
    def step(self):
        self.finish_grad_sync()
        self.step_count += 1
        b1, b2 = self.betas
        scale = self._clip_scale()
        bc1 = 1.0 - b1 ** self.step_count
        bc2 = 1.0 - b2 ** self.step_count
        n = self.shard_numel
        if self.fused_dp is not None:
            f, b = self.fused_dp, self.buckets[0]
            f["epoch"] += 1
            native.call("lb_dp_adamw", f["grads"], f["params"], f["flags"], f["counter"].data_ptr(),
                        self.master.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                        b.start + f["rank"] * b.shard_len, b.shard_len, f["n"], f["rank"], f["epoch"], self.lr, b1, b2,
                        self.eps, self.weight_decay, bc1, bc2, scale, f["grid"], native.stream_ptr())
            self._reset_buckets()
            return
        if self.native:
            native.call("lb_adamw", self.master.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                        self.grad_shard.data_ptr(), self.param_shard.data_ptr(), n, self.lr, b1, b2, self.eps,
                        self.weight_decay, bc1, bc2, scale, 0, native.stream_ptr())
        else:
            g = self.grad_shard.float() * scale
            ref.adamw_step(self.master, g, self.exp_avg, self.exp_avg_sq, self.lr, b1, b2, self.eps,
                           self.weight_decay, self.step_count)
            self.param_shard.copy_(self.master.to(self.param_shard.dtype))
        for b in self.buckets:
            src = self.param_shard[b.shard_off:b.shard_off + b.shard_len]
            dst = self.flat_params[b.start:b.end]
            if b.n == 1:
                if dst.data_ptr() != src.data_ptr():
                    dst.copy_(src)
            else:
                dist.all_gather_into_tensor(dst, src, group=b.group)
        self._reset_buckets()

    def zero_grad(self, set_to_none: bool = False):
        """One memset over the gradient arena (``.grad`` tensors stay views into it)."""
        self.flat_grads.zero_()
        for p in self.params:
            if p.grad is None or p.grad.data_ptr() != self.flat_grads.data_ptr() + p._arena_offset * self.flat_grads.element_size():
                p.grad = self.flat_grads[p._arena_offset:p._arena_offset + p.numel()].view(p.shape)
        self._reset_buckets()

    @torch.no_grad()
    def refresh_master_from_params(self):
        """Rebuild the fp32 master shard from the current parameters (after loading weights)."""
        for b in self.buckets:
            r = comm.group_rank(b.group)
            src = self.flat_params[b.start + r * b.shard_len: b.start + (r + 1) * b.shard_len]
            self.master[b.shard_off:b.shard_off + b.shard_len].copy_(src.float())

    # ---- checkpoint ---------------------------------------------------------------------------
    def state_dict(self):
        return {"step": self.step_count, "master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(),
                "exp_avg_sq": self.exp_avg_sq.cpu(), "lr": self.lr, "weight_decay": self.weight_decay,
                "betas": self.betas, "eps": self.eps, "shard_numel": self.shard_numel}

    def load_state_dict(self, sd):
        assert sd["shard_numel"] == self.shard_numel, "optimizer shard layout differs (re-shard not possible here)"
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
