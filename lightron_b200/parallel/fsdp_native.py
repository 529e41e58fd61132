"""Fully sharded data parallelism on peer memory (the CUDA bf16 engine behind ``distributed.fsdp``).

What the reference gets from PyTorch FSDP2 (``parallel/parallel_fsdp.py:115-183``: ``fully_shard`` per
transformer block, bf16 parameters, fp32 gradient reduction, ``reshard_after_forward``, wired in
``trainer.py:198-203``) is done here with our own kernels over NVLink peer memory:

* every transformer block is a unit whose parameters are one flat bf16 range; a rank keeps only
  its 1/n shard of it (bf16 for the gathers, fp32 master weights and Adam moments for the update);
* two peer-visible parameter slots and two gradient slots, each as large as the largest unit, are
  all the unsharded memory there is: unit i lives in slot i % 2 while it is computed, so autograd's
  saved weight views see the re-gathered values in backward, and unit i + 1 is gathered into the
  other slot while unit i computes (``lb_gather_into``: every rank stores its shard straight into
  every peer's slot; a slot is reused only after every rank has released its previous occupant);
* when the last gradient of a unit has been written (the weight-gradient GEMMs write straight into
  the gradient slot), ONE kernel on a side stream reads every replica's gradients of this rank's
  shard over NVLink, sums them in fp32, applies AdamW to the fp32 master shard and stores the new
  bf16 shard (``lb_fsdp_rs_adamw``): reduce-scatter, cast / scale and optimizer step fused, one
  launch per block, overlapped with the backward of the blocks below;
* with gradient accumulation the reduced gradient of the earlier micro-batches goes to an fp32
  accumulator shard (the reference reduces on every micro-batch too, ``:135-138``);
* embedding, final norm and output head form a root unit that stays gathered (as in the reference,
  ``:176-181``); expert parameters, which expert parallelism already divides over the same ranks,
  keep their local AdamW.

Scope: pp = 1, tp = 1, gradient clipping off, expert replica group of one rank; other layouts use
``parallel.fsdp`` (library collectives) or the default sharded-optimizer engine.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import native

_ALIGN = 128
_G = 32                     # CTAs of a parameter gather


def _up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class _Unit:
    def __init__(self, name: str, params: List[nn.Parameter], names: List[str], n: int):
        self.name, self.params, self.names = name, params, names
        self.shapes = [p.shape for p in params]
        self.offsets, total = [], 0
        for p in params:
            self.offsets.append(total)
            total += _up(p.numel(), _ALIGN)
        self.total = _up(total, _ALIGN * n)
        self.shard_len = self.total // n
        self.seen = set()              # parameters whose gradient has been written in the current backward
        self.gathered = False          # a gather into the unit's slot has been issued and not yet released
        self.gather_event = None
        self.rs_event = None


class NativeFSDP:
    """Engine + optimizer in one object (``zero_grad`` / ``step`` / ``set_requires_gradient_sync`` /
    ``state_dict``: the interface the trainer expects from its optimizer)."""

    def __init__(self, model: nn.Module, ctx, lr: float, weight_decay: float, betas=(0.9, 0.999), eps: float = 1e-8):
        import torch.distributed._symmetric_memory as symm_mem
        self.model, self.ctx = model, ctx
        self.lr, self.weight_decay, self.betas, self.eps = lr, weight_decay, tuple(betas), eps
        self.group = ctx.dpcp_group
        self.n, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        n = self.n
        self.step_count = 0
        self.sync_enabled = True
        self.grad_clip = 0.0
        dev = next(model.parameters()).device
        self.device = dev
        native.require()
        # ---- units ----
        blocks = list(model.layers.values())
        prefix_of = {id(m): nm for nm, m in model.named_modules()}
        seen = set()
        self.units: List[_Unit] = []
        self.expert_params: List[nn.Parameter] = []
        for blk in blocks:
            named = [(f"{prefix_of[id(blk)]}.{nm}", p) for nm, p in blk.named_parameters()]
            dense = [(nm, p) for nm, p in named if not getattr(p, "is_expert", False)]
            self.expert_params += [p for _, p in named if getattr(p, "is_expert", False)]
            seen.update(id(p) for _, p in named)
            self.units.append(_Unit(prefix_of[id(blk)], [p for _, p in dense], [nm for nm, _ in dense], n))
        rest = [(nm, p) for nm, p in model.named_parameters() if id(p) not in seen]
        self.root = _Unit("root", [p for _, p in rest], [nm for nm, _ in rest], n)
        self.blocks = blocks
        max_total = max(u.total for u in self.units)
        self.grid = native.sm_count() * 8
        # ---- peer-visible memory: flags | 2 param slots | 2 grad slots | root params | root grads ----
        flag_bytes = 16384
        self.slot_bytes = _up(max_total * 2, 4096)
        root_bytes = _up(self.root.total * 2, 4096)
        off = flag_bytes
        self.param_slot_off = [off, off + self.slot_bytes]
        off += 2 * self.slot_bytes
        self.grad_slot_off = [off, off + self.slot_bytes]
        off += 2 * self.slot_bytes
        self.root_param_off, self.root_grad_off = off, off + root_bytes
        off += 2 * root_bytes
        self.buf = symm_mem.empty(off, dtype=torch.uint8, device=dev)
        self.buf[:flag_bytes].zero_()
        hdl = symm_mem.rendezvous(self.buf, group=self.group)
        self._hdl = hdl
        base = int(getattr(hdl, "offset", 0))
        self.ptrs = [int(p) + base for p in hdl.buffer_ptrs]
        # flag layout (bytes): [0, 64) optimizer-kernel flags (16 words); per slot s at 1024 + s * 4096:
        # arrival table [n][G] u32, then at +2048 the release words [n]
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.epoch = 0
        self.slot_use = [0, 0]
        self.comm_stream = torch.cuda.Stream()
        # ---- shards ----
        with torch.no_grad():
            for i, u in enumerate(self.units + [self.root]):
                full = torch.zeros(u.total, dtype=torch.float32, device=dev)
                for p, o in zip(u.params, u.offsets):
                    full[o:o + p.numel()].copy_(p.data.reshape(-1).float())
                sh = full[self.rank * u.shard_len:(self.rank + 1) * u.shard_len]
                u.master = sh.clone()
                u.shard_bf16 = sh.to(torch.bfloat16)
                u.exp_avg = torch.zeros_like(u.master)
                u.exp_avg_sq = torch.zeros_like(u.master)
                u.acc = None
                if u is self.root:
                    pbuf = self._view(self.root_param_off, u.total)
                    gbuf = self._view(self.root_grad_off, u.total)
                    pbuf.copy_(full.to(torch.bfloat16))
                else:
                    pbuf = self._view(self.param_slot_off[i % 2], u.total)
                    gbuf = self._view(self.grad_slot_off[i % 2], u.total)
                u.pbuf, u.gbuf, u.slot = pbuf, gbuf, (i % 2)
                for p, o in zip(u.params, u.offsets):
                    p.data = pbuf[o:o + p.numel()].view(p.shape)
                    p.grad = gbuf[o:o + p.numel()].view(p.shape)
                    p._lb_direct_grad = True
                    hook = self._make_hook(u)
                    p.register_post_accumulate_grad_hook(hook)
                    p._lb_grad_hooks = (hook,)
        self.buf[self.root_grad_off:self.root_grad_off + root_bytes].zero_()
        # expert parameters: local flat arena + plain sharded-free AdamW
        self.exp_master = self.exp_m = self.exp_v = None
        if self.expert_params:
            assert dist.get_world_size(ctx.edpcp_group) == 1, "native FSDP needs every expert to live on exactly one rank"
            tot = sum(_up(p.numel(), _ALIGN) for p in self.expert_params)
            self.exp_flat = torch.zeros(tot, dtype=torch.bfloat16, device=dev)
            self.exp_grad = torch.zeros(tot, dtype=torch.bfloat16, device=dev)
            o = 0
            with torch.no_grad():
                for p in self.expert_params:
                    v = self.exp_flat[o:o + p.numel()].view(p.shape)
                    v.copy_(p.data)
                    p.data = v
                    p.grad = self.exp_grad[o:o + p.numel()].view(p.shape)
                    p._lb_direct_grad = True
                    o += _up(p.numel(), _ALIGN)
            self.exp_master = self.exp_flat.float()
            self.exp_m, self.exp_v = torch.zeros_like(self.exp_master), torch.zeros_like(self.exp_master)
            self.ep_scale = 1.0 / max(1, int(getattr(ctx, "ep_size", 1)))
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for i, (blk, u) in enumerate(zip(blocks, self.units)):
            self._wrap(blk, i)
        model._fsdp_native = self
        self.shard_numel = sum(u.shard_len for u in self.units) + self.root.shard_len

    # ---- plumbing -----------------------------------------------------------------------------
    def _view(self, off: int, numel: int) -> torch.Tensor:
        return self.buf[off:off + numel * 2].view(torch.bfloat16)

    def _arr(self, off: int):
        a = (ctypes.c_void_p * self.n)()
        for r in range(self.n):
            a[r] = self.ptrs[r] + off
        return a

    def _slot_flags(self, s: int):
        return 1024 + s * 4096

    def _make_hook(self, u: _Unit):
        n_params = sum(1 for p in u.params if p.requires_grad)

        def hook(p):
            # once per parameter and backward pass: an op that wrote the gradient straight into the
            # slot calls this by hand, and autograd may call it again for the same parameter
            if id(p) in u.seen:
                return
            u.seen.add(id(p))
            if len(u.seen) == n_params:
                u.seen = set()
                self._unit_backward_done(u)
        return hook

    def _wrap(self, blk: nn.Module, i: int) -> None:
        def pre_fwd(_m, _inp):
            self._need(i)
            if i + 1 < len(self.units):
                self._gather(i + 1)                    # prefetch into the other slot

        def post_fwd(_m, _inp, out):
            self._release(i)
            return out

        def pre_bwd(_m, _gout):
            self._need(i, for_backward=True)
            if i - 1 >= 0:
                self._gather(i - 1)

        blk.register_forward_pre_hook(pre_fwd)
        blk.register_forward_hook(post_fwd)
        blk.register_full_backward_pre_hook(pre_bwd)

    def _gather(self, i: int) -> None:
        """Issue the all-gather of unit i into its slot on the side stream (idempotent)."""
        u = self.units[i]
        if u.gathered:
            return
        s = u.slot
        self.slot_use[s] += 1
        cs = self.comm_stream
        cs.wait_stream(torch.cuda.current_stream())       # local readers of the slot's previous occupant are queued before this point
        with torch.cuda.stream(cs):
            fo = self._slot_flags(s)
            native.call("lb_gather_into", u.shard_bf16.data_ptr(), self._arr(self.param_slot_off[s]), self._arr(fo),
                        self.ptrs[self.rank] + fo + 2048, u.shard_len, self.n, self.rank, _G, self.slot_use[s],
                        cs.cuda_stream)
            u.gather_event = torch.cuda.Event()
            u.gather_event.record(cs)
        u.gathered = True
        u.use = self.slot_use[s]

    def _need(self, i: int, for_backward: bool = False) -> None:
        u = self.units[i]
        self._gather(i)
        torch.cuda.current_stream().wait_event(u.gather_event)
        if for_backward:
            # the gradient slot may still be read by the optimizer kernels of the unit two above
            j = i + 2
            if j < len(self.units) and self.units[j].rs_event is not None:
                torch.cuda.current_stream().wait_event(self.units[j].rs_event)
            u.gbuf.zero_()
            u.in_backward = True

    def _release(self, i: int) -> None:
        u = self.units[i]
        if not u.gathered:
            return
        fo = self._slot_flags(u.slot)
        native.call("lb_slot_release", self._arr(fo + 2048), self.n, self.rank, u.use, native.stream_ptr())
        u.gathered = False

    def _hyper(self):
        step = self.step_count + 1
        b1, b2 = self.betas
        return b1, b2, 1.0 - b1 ** step, 1.0 - b2 ** step

    def _launch_update(self, u: _Unit, grad_off: int, param_ptrs, push_all: int) -> None:
        do_update = 1 if self.sync_enabled else 0
        if not do_update and u.acc is None:
            u.acc = torch.zeros_like(u.master)
        b1, b2, bc1, bc2 = self._hyper()
        self.epoch += 1
        cs = self.comm_stream
        cs.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cs):
            native.call("lb_fsdp_rs_adamw", self._arr(grad_off), param_ptrs, self._arr(0), self.counter.data_ptr(),
                        u.master.data_ptr(), u.exp_avg.data_ptr(), u.exp_avg_sq.data_ptr(),
                        0 if u.acc is None else u.acc.data_ptr(), self.rank * u.shard_len, u.shard_len, self.n, self.rank,
                        self.epoch, self.lr, b1, b2, self.eps, self.weight_decay, bc1, bc2, 1.0, self.grid, do_update,
                        push_all, cs.cuda_stream)
            u.rs_event = torch.cuda.Event()
            u.rs_event.record(cs)

    def _unit_backward_done(self, u: _Unit) -> None:
        if u is self.root:
            return                                  # stepped in step(): its gradients complete last anyway
        i = self.units.index(u)
        self._release(i)
        # new bf16 parameters go to this rank's shard: pass a base such that base + shard_start is the shard
        arr = (ctypes.c_void_p * self.n)()
        for r in range(self.n):
            arr[r] = u.shard_bf16.data_ptr() - self.rank * u.shard_len * 2
        self._launch_update(u, self.grad_slot_off[u.slot], arr, 0)

    # ---- optimizer interface ---------------------------------------------------------------------
    def set_requires_gradient_sync(self, flag: bool) -> None:
        """False on all micro-batches but the last: reduced gradients go to the fp32 accumulator."""
        self.sync_enabled = bool(flag)

    def zero_grad(self, set_to_none: bool = False) -> None:
        self.root.gbuf.zero_()
        if self.expert_params:
            self.exp_grad.zero_()
        for u in self.units + [self.root]:
            u.seen = set()

    def finish_grad_sync(self) -> None:
        pass

    @torch.no_grad()
    def step(self) -> None:
        from ..ops import functional as OF
        OF.flush_wgrads()
        # root unit: reduce-scatter + AdamW + all-gather (it stays gathered)
        self._launch_update(self.root, self.root_grad_off, self._arr(self.root_param_off), 1)
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        if self.expert_params:
            b1, b2, bc1, bc2 = self._hyper()
            native.call("lb_adamw", self.exp_master.data_ptr(), self.exp_m.data_ptr(), self.exp_v.data_ptr(),
                        self.exp_grad.data_ptr(), self.exp_flat.data_ptr(), self.exp_master.numel(), self.lr, b1, b2,
                        self.eps, self.weight_decay, bc1, bc2, self.ep_scale, 0, native.stream_ptr())
        self.step_count += 1

    # ---- full tensors (checkpoints, tests) -------------------------------------------------------
    @torch.no_grad()
    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        torch.cuda.synchronize()
        for u in self.units + [self.root]:
            if u is self.root:
                full = u.pbuf                       # resident and refreshed by every step
            else:
                parts = [torch.empty_like(u.shard_bf16) for _ in range(self.n)]
                dist.all_gather(parts, u.shard_bf16, group=self.group)
                full = torch.cat(parts)
            for nm, o, shp in zip(u.names, u.offsets, u.shapes):
                out[nm] = full[o:o + int(torch.Size(shp).numel())].view(shp).cpu().clone()
        for nm, p in self.model.named_parameters():
            if getattr(p, "is_expert", False):
                out[nm] = p.detach().cpu().clone()
        return out

    @torch.no_grad()
    def load_full_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for u in self.units + [self.root]:
            full = torch.zeros(u.total, dtype=torch.float32, device=self.device)
            for nm, o, shp in zip(u.names, u.offsets, u.shapes):
                full[o:o + int(torch.Size(shp).numel())].copy_(sd[nm].reshape(-1).to(self.device).float())
            sh = full[self.rank * u.shard_len:(self.rank + 1) * u.shard_len]
            u.master.copy_(sh)
            u.shard_bf16.copy_(sh.to(torch.bfloat16))
            if u is self.root:
                u.pbuf.copy_(full.to(torch.bfloat16))
        for nm, p in self.model.named_parameters():
            if getattr(p, "is_expert", False) and nm in sd:
                p.copy_(sd[nm].to(self.device, p.dtype))
        if self.expert_params:
            self.exp_master.copy_(self.exp_flat.float())

    def refresh_master_from_params(self) -> None:
        pass                                        # load_full_state_dict already rebuilt the master shards

    def state_dict(self):
        def cat(attr):
            return torch.cat([getattr(u, attr).reshape(-1) for u in self.units + [self.root]]).cpu()
        sd = {"step": self.step_count, "master": cat("master"), "exp_avg": cat("exp_avg"), "exp_avg_sq": cat("exp_avg_sq"),
              "lr": self.lr, "weight_decay": self.weight_decay, "betas": self.betas, "eps": self.eps,
              "shard_numel": self.shard_numel}
        if self.expert_params:
            sd.update(exp_master=self.exp_master.cpu(), exp_m=self.exp_m.cpu(), exp_v=self.exp_v.cpu())
        return sd

    def load_state_dict(self, sd) -> None:
        assert sd["shard_numel"] == self.shard_numel, "optimizer shard layout differs"
        self.step_count = int(sd["step"])
        o = 0
        for u in self.units + [self.root]:
            u.master.copy_(sd["master"][o:o + u.shard_len])
            u.exp_avg.copy_(sd["exp_avg"][o:o + u.shard_len])
            u.exp_avg_sq.copy_(sd["exp_avg_sq"][o:o + u.shard_len])
            u.shard_bf16.copy_(u.master.to(torch.bfloat16))
            o += u.shard_len
        if self.expert_params and "exp_master" in sd:
            self.exp_master.copy_(sd["exp_master"]); self.exp_m.copy_(sd["exp_m"]); self.exp_v.copy_(sd["exp_v"])


def supported(model: nn.Module, ctx, dtype, grad_clip: float) -> Optional[str]:
    """None when the native engine can run this layout, else the reason it cannot."""
    if not (torch.cuda.is_available() and dtype == torch.bfloat16 and native.available()):
        return "needs CUDA, bf16 and the native library"
    if ctx.pp_size > 1 or ctx.tp_size > 1:
        return "pipeline / tensor parallel layouts use the library-collective FSDP engine"
    n = dist.get_world_size(ctx.dpcp_group) if dist.is_initialized() else 1
    if n < 2 or n > 8:
        return "needs 2..8 data-parallel ranks"
    if dist.get_backend(ctx.dpcp_group) != "nccl":
        return "needs the NCCL backend (peer memory)"
    if grad_clip > 0:
        return "gradient clipping needs the global norm before any block is stepped"
    if any(getattr(p, "is_expert", False) for p in model.parameters()) and dist.get_world_size(ctx.edpcp_group) != 1:
        return "expert parameters must not be replicated (ep_size == dp_size)"
    return None
