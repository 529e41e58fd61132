"""Context parallelism: zig-zag causal ring attention (forward + backward) and Ulysses.

Reference counterparts: ``parallel/parallel_cp.py`` (Ulysses: all-to-all of q,k,v from sequence
shards to head shards ``:206-208``, causal attention on the full sequence ``:224-229``, all-to-all
back ``:239``; autograd through ``SeqAllToAll`` ``:47-96``) and
``parallel/communication/ring_attention.py:10-119`` (forward-only, non-causal ring with an
online-softmax merge, never wired into the model).

Here the ring is causal with zig-zag load balance (rank r owns sequence chunks r and 2c-1-r, so
every ring step is either the local causal block or an unmasked half-size block and all ranks
do equal work), has a backward pass (dK/dV travel around the ring with their K/V block), is
GQA-aware (only KV heads move) and is used by the model.  Ulysses handles GQA by splitting KV
heads across ranks, replicating them when there are fewer KV heads than ranks.  Block math runs on
the flash-attention kernels (CUDA) or the fp32 oracle (CPU ranks).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import native, reference as ref
from . import comm


# ---- block primitives -----------------------------------------------------------------------------


def _block_fwd(q, k, v, causal: bool, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (o [B,Sq,hq,d] in q.dtype, lse [B,hq,Sq] fp32)."""
    if native.use_native(q):
        return OF.flash_fwd_native(q, k, v, causal, scale)
    return ref.attention(q, k, v, causal=causal, scale=scale, return_lse=True)


def _block_bwd(q, k, v, o, lse, do, causal: bool, scale: float):
    """Gradients of one (q-block, kv-block) pair given the FINAL output / log-sum-exp of the
    whole attention row (flash-attention backward identity: P = exp(S - lse))."""
    if native.use_native(q):
        return OF.flash_bwd_native(q, k, v, o, lse, do, causal, scale)
    B, Sq, hq, d = q.shape
    Sk, hkv = k.shape[1], k.shape[2]
    rep = hq // hkv
    qf = q.float().permute(0, 2, 1, 3).reshape(B, hkv, rep, Sq, d)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    dof = do.float().permute(0, 2, 1, 3).reshape(B, hkv, rep, Sq, d)
    of = o.float().permute(0, 2, 1, 3).reshape(B, hkv, rep, Sq, d)
    s = torch.einsum("bgrqd,bgkd->bgrqk", qf, kf) * scale
    if causal:
        mask = torch.arange(Sq, device=q.device)[:, None] + (Sk - Sq) >= torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.exp(s - lse.reshape(B, hkv, rep, Sq, 1))
    dv = torch.einsum("bgrqk,bgrqd->bgkd", p, dof)
    dp = torch.einsum("bgrqd,bgkd->bgrqk", dof, vf)
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.einsum("bgrqk,bgkd->bgrqd", ds, kf).reshape(B, hq, Sq, d).permute(0, 2, 1, 3)
    dk = torch.einsum("bgrqk,bgrqd->bgkd", ds, qf).permute(0, 2, 1, 3)
    return dq.to(q.dtype), dk.to(k.dtype), dv.permute(0, 2, 1, 3).to(v.dtype)


def _merge(o_acc, lse_acc, o_blk, lse_blk):
    """Online-softmax merge of two partial attention results (fp32 accumulators).
    o: [B,S,h,d], lse: [B,h,S]."""
    new = torch.logaddexp(lse_acc, lse_blk)
    wa = torch.exp(lse_acc - new).transpose(1, 2).unsqueeze(-1)
    wb = torch.exp(lse_blk - new).transpose(1, 2).unsqueeze(-1)
    return o_acc * wa + o_blk.float() * wb, new


def _ring_exchange(send: torch.Tensor, group):
    """Send to the next rank of the ring, receive from the previous one.  Returns (recv, reqs)."""
    n, r = dist.get_world_size(group), dist.get_rank(group)
    nxt = dist.get_global_rank(group, (r + 1) % n)
    prv = dist.get_global_rank(group, (r - 1) % n)
    recv = torch.empty_like(send)
    ops = [dist.P2POp(dist.isend, send, nxt, group), dist.P2POp(dist.irecv, recv, prv, group)]
    if r % 2:                       # alternate order so that unbatched backends cannot deadlock
        ops.reverse()
    return recv, dist.batch_isend_irecv(ops)


def _wait(reqs):
    for q in reqs:
        q.wait()


# ---- zig-zag ring attention -----------------------------------------------------------------------


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, scale):
        c, r = dist.get_world_size(group), dist.get_rank(group)
        B, S, hq, d = q.shape
        n = S // 2
        kv = torch.stack((k, v)).contiguous()
        o_acc = torch.zeros(B, S, hq, d, dtype=torch.float32, device=q.device)
        lse_acc = torch.full((B, hq, S), float("-inf"), dtype=torch.float32, device=q.device)
        for step in range(c):
            j = (r - step) % c
            if step + 1 < c:
                kv_next, reqs = _ring_exchange(kv, group)
            kb, vb = kv[0], kv[1]
            if step == 0:
                o_b, l_b = _block_fwd(q, kb, vb, True, scale)
                o_acc, lse_acc = _merge(o_acc, lse_acc, o_b, l_b)
            elif j < r:
                o_b, l_b = _block_fwd(q, kb[:, :n], vb[:, :n], False, scale)
                o_acc, lse_acc = _merge(o_acc, lse_acc, o_b, l_b)
            else:
                o_b, l_b = _block_fwd(q[:, n:], kb, vb, False, scale)
                o2, l2 = _merge(o_acc[:, n:], lse_acc[:, :, n:], o_b, l_b)
                o_acc = torch.cat((o_acc[:, :n], o2), dim=1)
                lse_acc = torch.cat((lse_acc[:, :, :n], l2), dim=2)
            if step + 1 < c:
                _wait(reqs)
                kv = kv_next
        o = o_acc.to(q.dtype)
        ctx.save_for_backward(q, k, v, o, lse_acc)
        ctx.group, ctx.scale = group, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        group, scale = ctx.group, ctx.scale
        c, r = dist.get_world_size(group), dist.get_rank(group)
        B, S, hq, d = q.shape
        n = S // 2
        do = do.contiguous()
        kv = torch.stack((k, v)).contiguous()
        dq = torch.zeros(B, S, hq, d, dtype=torch.float32, device=q.device)
        dkv = torch.zeros((2,) + tuple(k.shape), dtype=torch.float32, device=q.device)
        dkv_recv, dkv_reqs = None, None
        lse_hi = lse[:, :, n:].contiguous()
        for step in range(c):
            j = (r - step) % c
            if step + 1 < c:
                kv_next, reqs = _ring_exchange(kv, group)
            kb, vb = kv[0], kv[1]
            if step == 0:
                dq_b, dk_b, dv_b = _block_bwd(q, kb, vb, o, lse, do, True, scale)
                dq += dq_b.float()
                part = torch.stack((dk_b, dv_b)).float()
            elif j < r:
                dq_b, dk_b, dv_b = _block_bwd(q, kb[:, :n], vb[:, :n], o, lse, do, False, scale)
                dq += dq_b.float()
                part = torch.zeros_like(dkv)
                part[0, :, :n] = dk_b.float()
                part[1, :, :n] = dv_b.float()
            else:
                dq_b, dk_b, dv_b = _block_bwd(q[:, n:], kb, vb, o[:, n:], lse_hi, do[:, n:], False, scale)
                dq[:, n:] += dq_b.float()
                part = torch.stack((dk_b, dv_b)).float()
            if step > 0:
                _wait(dkv_reqs)
                dkv = dkv_recv
            dkv = dkv + part
            dkv_recv, dkv_reqs = _ring_exchange(dkv.contiguous(), group)
            if step + 1 < c:
                _wait(reqs)
                kv = kv_next
        _wait(dkv_reqs)
        return dq.to(q.dtype), dkv_recv[0].to(k.dtype), dkv_recv[1].to(v.dtype), None, None


def ring_attention(q, k, v, group, scale: Optional[float] = None) -> torch.Tensor:
    """Causal attention over a sequence that is zig-zag sharded across ``group``.
    q [B, S_local, hq, d], k/v [B, S_local, hkv, d]; local rows are [chunk r | chunk 2c-1-r]."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if comm.group_size(group) == 1:
        return OF.flash_attention(q, k, v, True, scale)
    return _RingAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), group, scale)


# ---- Ulysses ----------------------------------------------------------------------------------------


def seq_gather_head_scatter(x: torch.Tensor, group) -> torch.Tensor:
    """[B, S/c, h, d] -> [B, S, h/c, d] (sequence is contiguously sharded)."""
    c = comm.group_size(group)
    B, Sl, h, d = x.shape
    t = x.reshape(B, Sl, c, h // c, d).permute(2, 0, 1, 3, 4).contiguous()
    t = comm.all_to_all_rows(t.view(c * B, Sl, h // c, d), group)
    return t.view(c, B, Sl, h // c, d).permute(1, 0, 2, 3, 4).reshape(B, c * Sl, h // c, d)


def seq_scatter_head_gather(x: torch.Tensor, group) -> torch.Tensor:
    """[B, S, h/c, d] -> [B, S/c, h, d]."""
    c = comm.group_size(group)
    B, S, hl, d = x.shape
    Sl = S // c
    t = x.reshape(B, c, Sl, hl, d).permute(1, 0, 2, 3, 4).contiguous()
    t = comm.all_to_all_rows(t.view(c * B, Sl, hl, d), group)
    return t.view(c, B, Sl, hl, d).permute(1, 2, 0, 3, 4).reshape(B, Sl, c * hl, d)


def ulysses_attention(q, k, v, group, scale: Optional[float] = None) -> torch.Tensor:
    """q [B, S/c, hq, d] (RoPE already applied at global positions), k/v [B, S/c, hkv, d]."""
    c = comm.group_size(group)
    hq, hkv = q.shape[2], k.shape[2]
    assert hq % c == 0, f"Ulysses needs local q heads ({hq}) divisible by cp ({c})"
    if hkv % c:
        assert c % hkv == 0, f"Ulysses needs kv heads ({hkv}) to divide or be divisible by cp ({c})"
        rep = c // hkv
        k = k.repeat_interleave(rep, dim=2)
        v = v.repeat_interleave(rep, dim=2)
    qg = seq_gather_head_scatter(q, group)
    kg = seq_gather_head_scatter(k, group)
    vg = seq_gather_head_scatter(v, group)
    o = OF.flash_attention(qg, kg, vg, True, scale)
    return seq_scatter_head_gather(o, group)


# ---- model entry -------------------------------------------------------------------------------------


def context_parallel_attention(qkv, cos, sin, positions, B, S, hq, hkv, d, group, mode: str) -> torch.Tensor:
    """qkv [B*S_local, (hq+2hkv)*d] -> attention output [B*S_local, hq*d].
    ``positions`` are the global positions of the local rows (zig-zag for ring, contiguous for
    Ulysses); RoPE is applied locally before any exchange."""
    T = B * S
    if mode == "ulysses" and comm.group_size(group) > 1:
        from . import ulysses_fused
        if ulysses_fused.fused_ok(qkv, group, hq, hkv, d):
            # exchange, layout change and RoPE in one kernel per direction (peer stores over NVLink)
            return ulysses_fused.ulysses_attention_qkv(qkv, cos, sin, positions, B, S, hq, hkv, d, group)
    q, k, v = qkv.view(T, -1).split([hq * d, hkv * d, hkv * d], dim=-1)
    q = OF.rope(q.reshape(B, S, hq, d), cos, sin, positions)
    k = OF.rope(k.reshape(B, S, hkv, d), cos, sin, positions)
    v = v.reshape(B, S, hkv, d).contiguous()
    if mode == "ring":
        o = ring_attention(q, k, v, group)
    elif mode == "allgather":
        from .cp_fused import allgather_kv_attention
        o = allgather_kv_attention(q, k, v, group, positions=positions)
    elif mode == "ulysses":
        o = ulysses_attention(q, k, v, group)
    else:
        raise ValueError(f"unknown cp_mode {mode}")
    return o.reshape(T, hq * d)


class ContextParallelAttention(torch.nn.Module):
    """API-parity wrapper (reference: parallel/parallel_cp.py:104-245): wraps an ``Attention``
    module so that its forward runs context-parallel.  The wrapped module's parameters keep their
    plain names (the reference's wrapper adds ``.local_attn.`` to every key)."""

    def __init__(self, local_attn, args=None, group="auto", mode: Optional[str] = None):
        super().__init__()
        from .. import mesh
        object.__setattr__(self, "_inner", local_attn)
        local_attn.cp_group = mesh.get_cp_group() if group == "auto" else group
        if mode is not None:
            local_attn.cp_mode = mode

    def forward(self, *a, **kw):
        return self._inner(*a, **kw)
