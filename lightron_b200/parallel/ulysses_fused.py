"""Ulysses context parallelism with the all-to-all, the layout change and RoPE in one kernel.

The reference (``parallel/parallel_cp.py:154-245``) runs, per attention layer and direction, three
``dist.all_to_all`` calls on lists of chunks (q, k, v: sequence shards -> head shards, ``:206-208``)
and one back (``:239``), each surrounded by ``split`` / ``cat`` / ``transpose`` / ``contiguous`` copies,
with RoPE as separate complex multiplies (``:219``).  Here ``lb_ulysses_a2a`` reads the fused QKV
projection output where the GEMM left it, rotates q and k on the fly and stores every head straight
into the row and head position it has on the rank that will attend over it (16-byte peer stores over
NVLink); after attention the same kernel stores every output row into the ``[tokens, heads * d]``
matrix of its owner, which is the operand of the ``wo`` GEMM as it is.  Backward uses the same two
directions on the gradients (and the inverse rotation).  GQA: KV heads are split over the ranks, or,
with fewer KV heads than ranks, each rank receives one copy of its KV head and the gradients of the
copies are summed.

CPU ranks and unsupported shapes keep ``cp.ulysses_attention`` (library all-to-all).
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import native

_G = 64


class _Pool:
    """Peer-visible buffers of one CP group for one problem size: a flag table, per attention layer a
    slot (q, k, v as attended and the returned output: all four stay alive until the layer's
    backward), and two alternating sets of gradient buffers."""

    def __init__(self, group, B, Sl, hq, hkv, d, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.symm = symm_mem
        self.group = group
        self.n, self.rank = dist.get_world_size(group), dist.get_rank(group)
        c = self.n
        self.B, self.Sl, self.hq, self.hkv, self.d = B, Sl, hq, hkv, d
        self.S = c * Sl
        self.hql = hq // c
        self.rep = 1 if hkv % c == 0 else c // hkv
        self.hkl = hkv // c if self.rep == 1 else 1
        self.device = device
        self.flags, self.flag_ptrs = self._alloc(self.n * _G * 4 + 256, zero=True)
        self.call = 0
        self.free: List[dict] = []
        self.bwd_sets = [self._grad_set(), self._grad_set()]
        self.bwd_calls = 0
        self.nograd_slots: List[dict] = []
        self.nograd_calls = 0

    def _alloc(self, nbytes, zero=False):
        t = self.symm.empty((nbytes + 255) // 256 * 256, dtype=torch.uint8, device=self.device)
        if zero:
            t.zero_()
        hdl = self.symm.rendezvous(t, group=self.group)
        off = int(getattr(hdl, "offset", 0))
        ptrs = [int(p) + off for p in hdl.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        return t, ptrs

    def _buf(self, *shape):
        numel = 1
        for s in shape:
            numel *= s
        t, ptrs = self._alloc(numel * 2)
        return {"t": t[: numel * 2].view(torch.bfloat16).view(*shape), "ptrs": ptrs}

    def _slot(self):
        B, S, Sl, d = self.B, self.S, self.Sl, self.d
        return {"q": self._buf(B, S, self.hql, d), "k": self._buf(B, S, self.hkl, d), "v": self._buf(B, S, self.hkl, d),
                "o": self._buf(B * Sl, self.hq * d)}

    def _grad_set(self):
        B, S, Sl, d = self.B, self.S, self.Sl, self.d
        hkv_x = self.hkv * self.rep if self.rep > 1 else self.hkv            # expanded KV heads coming back
        return {"do": self._buf(B, S, self.hql, d), "dq": self._buf(B * Sl, self.hq * d),
                "dk": self._buf(B * Sl, hkv_x * d), "dv": self._buf(B * Sl, hkv_x * d)}

    def acquire(self, keep: bool) -> dict:
        """A slot for one attention layer.  With autograd the slot lives until the layer's backward has
        run; without, two slots alternate (a peer is never two layers ahead)."""
        if not keep:
            if len(self.nograd_slots) < 2:
                self.nograd_slots.append(self._slot())
            self.nograd_calls += 1
            return self.nograd_slots[self.nograd_calls % 2]
        return self.free.pop() if self.free else self._slot()

    def release(self, slot: dict) -> None:
        self.free.append(slot)

    def arr(self, ptrs):
        a = (ctypes.c_void_p * self.n)()
        for r in range(self.n):
            a[r] = ptrs[r]
        return a

    def a2a(self, mode, src, src_ld, col0, dst, dst_ld, dst_col0, H, hl, rep, cos=None, sin=None, pos=None, inverse=False):
        self.call += 1
        native.call("lb_ulysses_a2a", mode, src.data_ptr(), src_ld, col0, dst_ld, dst_col0, self.arr(dst["ptrs"]),
                    self.arr(self.flag_ptrs), native.ptr(cos), native.ptr(sin), native.ptr(pos), int(inverse), self.B, self.Sl,
                    H, hl, self.d, rep, self.n, self.rank, _G, self.call, native.stream_ptr())


_POOLS: Dict[tuple, _Pool] = {}


def _pool(group, B, Sl, hq, hkv, d, device) -> _Pool:
    key = (id(group), B, Sl, hq, hkv, d)
    p = _POOLS.get(key)
    if p is None:
        p = _POOLS[key] = _Pool(group, B, Sl, hq, hkv, d, device)
    return p


def fused_ok(qkv: torch.Tensor, group, hq: int, hkv: int, d: int) -> bool:
    if not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and native.available()):
        return False
    from . import symm
    c = dist.get_world_size(group)
    return symm.supported(group) and d in (64, 128) and hq % c == 0 and (hkv % c == 0 or c % hkv == 0)


class _UlyssesAttention(torch.autograd.Function):
    """qkv [B*Sl, (hq+2hkv)*d] (this rank's contiguous sequence shard) -> attention output
    [B*Sl, hq*d] over the whole sequence."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, group, B, Sl, hq, hkv, d, scale):
        pool = _pool(group, B, Sl, hq, hkv, d, qkv.device)
        W = (hq + 2 * hkv) * d
        qkv2 = qkv.view(B * Sl, W)
        keep = bool(ctx.needs_input_grad[0])      # (grad mode itself is off inside forward)
        slot = pool.acquire(keep)
        ld = qkv2.stride(0)
        # sequence shards -> head shards, q and k rotated on the way
        pool.a2a(0, qkv2, ld, 0, slot["q"], 0, 0, hq, pool.hql, 1, cos, sin, positions)
        pool.a2a(0, qkv2, ld, hq * d, slot["k"], 0, 0, hkv, pool.hkl, pool.rep, cos, sin, positions)
        pool.a2a(0, qkv2, ld, (hq + hkv) * d, slot["v"], 0, 0, hkv, pool.hkl, pool.rep)
        qg, kg, vg = slot["q"]["t"], slot["k"]["t"], slot["v"]["t"]
        o, lse = OF.flash_fwd_native(qg, kg, vg, True, scale)
        # head shards -> sequence shards, straight into the [tokens, heads * d] operand of the wo GEMM
        pool.a2a(1, o, 0, 0, slot["o"], hq * d, 0, 0, pool.hql, 1)
        ctx.save_for_backward(o, lse, cos, sin, positions)
        ctx.slot, ctx.pool, ctx.dims = slot, pool, (B, Sl, hq, hkv, d, scale)
        ctx.keep = keep
        # a fresh view object per call: the buffer's own tensor object would carry the autograd
        # history of the layer (or step) that used the slot before
        return slot["o"]["t"].view(B * Sl, hq * d)

    @staticmethod
    def backward(ctx, dout):
        o, lse, cos, sin, positions = ctx.saved_tensors
        slot, pool = ctx.slot, ctx.pool
        B, Sl, hq, hkv, d, scale = ctx.dims
        gs = pool.bwd_sets[pool.bwd_calls % 2]
        pool.bwd_calls += 1
        dout = dout.contiguous()
        # gradient of the output: sequence shards -> head shards
        pool.a2a(0, dout.view(B * Sl, hq * d), hq * d, 0, gs["do"], 0, 0, hq, pool.hql, 1)
        qg, kg, vg = slot["q"]["t"], slot["k"]["t"], slot["v"]["t"]
        dqg, dkg, dvg = OF.flash_bwd_native(qg, kg, vg, o, lse, gs["do"]["t"], True, scale)
        # head shards -> sequence shards
        hkv_x = hkv * pool.rep if pool.rep > 1 else hkv
        pool.a2a(1, dqg, 0, 0, gs["dq"], hq * d, 0, 0, pool.hql, 1)
        pool.a2a(1, dkg, 0, 0, gs["dk"], hkv_x * d, 0, 0, pool.hkl, 1)
        pool.a2a(1, dvg, 0, 0, gs["dv"], hkv_x * d, 0, 0, pool.hkl, 1)
        W = (hq + 2 * hkv) * d
        dqkv = torch.empty(B * Sl, W, dtype=dout.dtype, device=dout.device)
        dqkv[:, :hq * d].copy_(gs["dq"]["t"])
        if pool.rep > 1:                                 # the copies of a KV head add up
            dqkv[:, hq * d:(hq + hkv) * d].copy_(gs["dk"]["t"].view(B * Sl, hkv, pool.rep, d).float().sum(2).view(B * Sl, hkv * d))
            dqkv[:, (hq + hkv) * d:].copy_(gs["dv"]["t"].view(B * Sl, hkv, pool.rep, d).float().sum(2).view(B * Sl, hkv * d))
        else:
            dqkv[:, hq * d:(hq + hkv) * d].copy_(gs["dk"]["t"])
            dqkv[:, (hq + hkv) * d:].copy_(gs["dv"]["t"])
        OF._rope_native_(dqkv, cos, sin, positions, Sl, hq + hkv, d, True)     # un-rotate the q and k gradients
        if ctx.keep:
            pool.release(slot)
        return dqkv.view(B * Sl, W), None, None, None, None, None, None, None, None, None, None


def ulysses_attention_qkv(qkv, cos, sin, positions, B, Sl, hq, hkv, d, group, scale: Optional[float] = None):
    """The fused QKV projection output of a contiguously sharded sequence -> attention output
    [B*Sl, hq*d]; ``positions`` [Sl] int32: global positions of the local rows."""
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if positions is not None and positions.dtype != torch.int32:
        positions = positions.to(torch.int32)
    return _UlyssesAttention.apply(qkv, cos, sin, positions, group, B, Sl, hq, hkv, d, scale)
