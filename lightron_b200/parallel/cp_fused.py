"""Context parallelism with the K/V exchange inside the attention kernel ("all-gather KV").

Every rank owns two zig-zag chunks of the sequence (r and 2c-1-r).  Instead of c ring steps
with an online-softmax merge after each, the forward attention launch itself contains mover CTAs
that PUSH this rank's K/V chunks into every peer's gather buffer over NVLink (coalesced peer
stores, one counter per 128-key block), while its attention CTAs consume key blocks as their
counters arrive (``lb_flash_fwd_cp``).  Each query chunk then needs exactly one causal attention
over a key prefix: chunk r over keys [0, (r+1)n), chunk 2c-1-r over keys [0, (2c-r)n); both are
plain bottom-right-aligned causal problems, so there is no partial-result merging at all.
GQA keeps the exchanged bytes small (only KV heads move) and 180 GB of HBM makes the gathered
prefix affordable as the tensor saved for backward.  Backward runs the two attention backwards
and reduce-scatters dK/dV to the owners of the chunks.

The reference has no counterpart (its ring attention is a forward-only non-causal demo,
parallel/communication/ring_attention.py:10-119); the north-star asks for the exchange to be
fused into the attention kernel, which this is.  CPU ranks and unsupported shapes take an
all-gather + oracle-attention path with the same math.
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import native, reference as ref
from . import comm

_MOVER_CTAS = 16
_WARPS = 10                      # warps per mover CTA (320 threads): each adds 1 per K and per V block


class _Workspace:
    def __init__(self, group, B: int, S: int, row_elems: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.key = (B, S, row_elems)
        self.n, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.fpb = S // 128
        self.flag_bytes = (2 * B * self.fpb * 4 + 255) // 256 * 256
        self.buf_bytes = (B * S * row_elems * 2 + 255) // 256 * 256
        total = self.flag_bytes + 4 * self.buf_bytes            # 2 slots x (K, V)
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf[: self.flag_bytes].zero_()
        hdl = symm_mem.rendezvous(self.buf, group=group)
        off = int(getattr(hdl, "offset", 0))
        self.ptrs = [int(p) + off for p in hdl.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self.calls = 0
        self.uses = [0, 0]

    def arr(self, off: int):
        a = (ctypes.c_void_p * self.n)()
        for r in range(self.n):
            a[r] = self.ptrs[r] + off
        return a

    def flag_off(self, slot: int, B: int) -> int:
        return slot * B * self.fpb * 4

    def k_off(self, slot: int) -> int:
        return self.flag_bytes + (2 * slot) * self.buf_bytes

    def v_off(self, slot: int) -> int:
        return self.flag_bytes + (2 * slot + 1) * self.buf_bytes

    def view(self, off: int, B: int, S: int, hkv: int, d: int) -> torch.Tensor:
        return self.buf[off:off + B * S * hkv * d * 2].view(torch.bfloat16).view(B, S, hkv, d)


_WS: Dict[int, _Workspace] = {}


def _workspace(group, B, S, row_elems, device) -> _Workspace:
    ws = _WS.get(id(group))
    if ws is None or ws.key != (B, S, row_elems):
        if ws is not None:
            torch.cuda.synchronize()
            dist.barrier(group=group)
        ws = _WS[id(group)] = _Workspace(group, B, S, row_elems, device)
    return ws


def fused_ok(q: torch.Tensor, group) -> bool:
    if not (q.is_cuda and q.dtype == torch.bfloat16 and native.available()):
        return False
    from . import symm
    B, Sl, hq, d = q.shape
    return symm.supported(group) and d in (64, 128) and Sl % 256 == 0


def _bwd_call(q, kbuf, vbuf, Sk, kv_brows, o, lse, do, scale):
    """Attention backward of q [B,n,hq,d] over the first Sk keys of every batch of kbuf/vbuf."""
    B, Sq, hq, d = q.shape
    hkv = kbuf.shape[2]
    dq = torch.empty_like(q)
    dk = torch.empty(B, Sk, hkv, d, dtype=q.dtype, device=q.device)
    dv = torch.empty_like(dk)
    delta = torch.empty(B, hq, Sq, dtype=torch.float32, device=q.device)
    dq_acc = torch.zeros(B * hq * ((Sq + 127) // 128) * 128 * d, dtype=torch.float32, device=q.device)
    native.call("lb_flash_bwd_cp", q.data_ptr(), kbuf.data_ptr(), vbuf.data_ptr(), o.data_ptr(), do.data_ptr(),
                lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                B, Sq, Sk, kv_brows, hq, hkv, d, q.stride(1), kbuf.stride(1), vbuf.stride(1), o.stride(1), do.stride(1),
                dq.stride(1), dk.stride(1), dv.stride(1), float(scale), 1, native.stream_ptr())
    return dq, dk, dv


class _AllGatherKVAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, scale):
        c, r = dist.get_world_size(group), dist.get_rank(group)
        B, Sl, hq, d = q.shape
        hkv = k.shape[2]
        n = Sl // 2
        S = 2 * c * n
        ws = _workspace(group, B, S, hkv * d, q.device)
        slot = ws.calls % 2
        ws.calls += 1
        ws.uses[slot] += 1
        target = ws.uses[slot] * 2 * _WARPS
        k, v = k.contiguous(), v.contiguous()
        qa, qb = q[:, :n].contiguous(), q[:, n:].contiguous()
        sk_a, sk_b = (r + 1) * n, (2 * c - r) * n
        kg = ws.view(ws.k_off(slot), B, S, hkv, d)
        vg = ws.view(ws.v_off(slot), B, S, hkv, d)
        flags_local = ws.ptrs[ws.rank] + ws.flag_off(slot, B)
        outs = []
        for (qq, sk, n_mov) in ((qb, sk_b, _MOVER_CTAS), (qa, sk_a, 0)):      # the long prefix carries the movers
            o = torch.empty_like(qq)
            lse = torch.empty(B, hq, n, dtype=torch.float32, device=q.device)
            native.call("lb_flash_fwd_cp", qq.data_ptr(), kg.data_ptr(), vg.data_ptr(), o.data_ptr(), lse.data_ptr(),
                        B, n, sk, S, hq, hkv, d, qq.stride(1), o.stride(1), float(scale), 1, flags_local, target, n_mov,
                        k.data_ptr(), v.data_ptr(), k.stride(1), v.stride(1), c, r, ws.arr(ws.k_off(slot)),
                        ws.arr(ws.v_off(slot)), ws.arr(ws.flag_off(slot, B)), n, native.stream_ptr())
            outs.append((o, lse))
        (ob, lb), (oa, la) = outs
        k_keep = kg[:, :sk_b].clone()            # the workspace slot is recycled two calls later
        v_keep = vg[:, :sk_b].clone()
        ctx.save_for_backward(qa, qb, k_keep, v_keep, oa, ob, la, lb)
        ctx.meta = (group, scale, c, r, n, sk_a, sk_b)
        return torch.cat((oa, ob), dim=1)

    @staticmethod
    def backward(ctx, do):
        qa, qb, kk, vk, oa, ob, la, lb = ctx.saved_tensors
        group, scale, c, r, n, sk_a, sk_b = ctx.meta
        B, _, hkv, d = kk.shape
        do_a, do_b = do[:, :n].contiguous(), do[:, n:].contiguous()
        dqa, dka, dva = _bwd_call(qa, kk, vk, sk_a, sk_b, oa, la, do_a, scale)
        dqb, dkb, dvb = _bwd_call(qb, kk, vk, sk_b, sk_b, ob, lb, do_b, scale)
        S = 2 * c * n
        dkv = torch.zeros(2, B, S, hkv, d, dtype=torch.float32, device=do.device)
        dkv[0, :, :sk_b] += dkb.float()
        dkv[1, :, :sk_b] += dvb.float()
        dkv[0, :, :sk_a] += dka.float()
        dkv[1, :, :sk_a] += dva.float()
        # rows of the owner j are chunks j and 2c-1-j: bring them together, then reduce-scatter
        idx = torch.tensor([x for j in range(c) for x in (j, 2 * c - 1 - j)], device=do.device)
        by_owner = dkv.view(2, B, 2 * c, n, hkv, d).index_select(2, idx).view(2, B, c, 2 * n, hkv, d)
        by_owner = by_owner.permute(2, 0, 1, 3, 4, 5).contiguous()                 # [c, 2, B, 2n, hkv, d]
        mine = comm.reduce_scatter_rows(by_owner.view(c, -1), group).view(2, B, 2 * n, hkv, d)
        return torch.cat((dqa, dqb), dim=1), mine[0].to(do.dtype), mine[1].to(do.dtype), None, None


def _oracle_path(q, k, v, group, scale, positions):
    """Same math with library collectives and the PyTorch attention (CPU ranks, odd shapes)."""
    c, r = comm.group_size(group), comm.group_rank(group)
    B, Sl, hkv, d = k.shape
    n = Sl // 2

    def gather(t):                                   # [B, Sl, h, d] -> [B, S, h, d] in sequence order
        rows = t.permute(1, 0, 2, 3).reshape(Sl, -1)
        full = comm.gather_rows(rows.contiguous(), group).view(c, 2, n, B, hkv, d)
        order = [(j, 0) if j < c else (2 * c - 1 - j, 1) for j in range(2 * c)]
        chunks = [full[a, b] for a, b in order]
        return torch.cat(chunks, dim=0).permute(1, 0, 2, 3)

    kf, vf = gather(k), gather(v)
    if positions is None:
        from ..data import cp_slice_indices
        positions = cp_slice_indices(2 * c * n, c, r, "zigzag").to(q.device)
    return ref.attention(q, kf, vf, causal=True, scale=scale, q_pos=positions.long(),
                         k_pos=torch.arange(2 * c * n, device=q.device))


def allgather_kv_attention(q, k, v, group, scale: Optional[float] = None, positions=None) -> torch.Tensor:
    """Causal attention over a zig-zag sharded sequence.  q [B, S_local, hq, d], k/v [B, S_local, hkv, d]
    (RoPE already applied); local rows are [chunk r | chunk 2c-1-r]."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if comm.group_size(group) == 1:
        return OF.flash_attention(q, k, v, True, scale)
    if fused_ok(q, group):
        return _AllGatherKVAttention.apply(q.contiguous(), k, v, group, scale)
    return _oracle_path(q, k, v, group, scale, positions)
