"""Context parallelism with the K/V exchange inside the attention kernel ("all-gather KV").

Every rank owns two zig-zag chunks of the sequence (r and 2c-1-r).  Instead of c ring steps
with an online-softmax merge after each, the forward attention launch itself contains mover CTAs
that PUSH this rank's K/V chunks into every peer's gather buffer over NVLink (coalesced peer
stores, one counter per 128-key block), while its attention CTAs consume key blocks as their
counters arrive (``lb_flash_fwd_cp``).  Each query chunk then needs exactly one causal attention
over a key prefix: chunk r over keys [0, (r+1)n), chunk 2c-1-r over keys [0, (2c-r)n); both are
plain bottom-right-aligned causal problems, so there is no partial-result merging at all.
GQA keeps the exchanged bytes small (only KV heads move) and 180 GB of HBM makes the gathered
prefix affordable as the tensor saved for backward.  Backward runs the two attention backwards, which
store their dK / dV partials into peer-visible buffers, and one kernel (``lb_cp_dkv_reduce``) in which
every owner reads and sums the partials that cover its chunks.

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


class _Workspace:
    def __init__(self, group, B: int, S: int, row_elems: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.key = (B, S, row_elems)
        self.n, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.fpb = S // 128
        self.flag_bytes = (2 * B * self.fpb * 4 + 255) // 256 * 256
        self.buf_bytes = (B * S * row_elems * 2 + 255) // 256 * 256
        # 2 slots x (K, V) for the forward exchange, then 2 parities x (dK a, dK b, dV a, dV b) partials of
        # the backward, then the ready words of the dK / dV reduction
        self.grad_off0 = self.flag_bytes + 4 * self.buf_bytes
        self.ready_off = self.grad_off0 + 8 * self.buf_bytes
        total = self.ready_off + 256
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf[self.ready_off:].zero_()
        self.buf[: self.flag_bytes].zero_()
        hdl = symm_mem.rendezvous(self.buf, group=group)
        off = int(getattr(hdl, "offset", 0))
        self.ptrs = [int(p) + off for p in hdl.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self.calls = 0
        self.uses = [0, 0]
        self.bwd_calls = 0

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

    def grad_off(self, parity: int, which: int) -> int:
        """which: 0 dK of call a, 1 dK of call b, 2 dV of call a, 3 dV of call b."""
        return self.grad_off0 + (4 * parity + which) * self.buf_bytes

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


def _bwd_call(q, kbuf, vbuf, Sk, kv_brows, o, lse, do, scale, dk=None, dv=None):
    """Attention backward of q [B,n,hq,d] over the first Sk keys of every batch of kbuf/vbuf.
    dk / dv [B, Sk, hkv, d] may be views of peer-visible memory."""
    B, Sq, hq, d = q.shape
    hkv = kbuf.shape[2]
    dq = torch.empty_like(q)
    if dk is None:
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
        target = ws.uses[slot] * 2 * native.require().lb_flash_fwd_cp_mover_warps()   # every mover warp counts K and V
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
        # The backward kernels store their dK / dV partials straight into peer-visible buffers; one
        # kernel then lets every owner read the partials that cover its two chunks, sum them in fp32
        # and keep its rows (no full-sequence fp32 buffer, no library reduce-scatter).  Two sets of
        # buffers alternate: a rank can reach the layer after next only after every peer has finished
        # reading this layer's partials.
        ws = _WS[id(group)]
        par = ws.bwd_calls % 2
        ws.bwd_calls += 1
        views = []
        for which, sk in ((0, sk_a), (1, sk_b), (2, sk_a), (3, sk_b)):
            off = ws.grad_off(par, which)
            views.append(ws.buf[off:off + B * sk * hkv * d * 2].view(torch.bfloat16).view(B, sk, hkv, d))
        dqa, _, _ = _bwd_call(qa, kk, vk, sk_a, sk_b, oa, la, do_a, scale, views[0], views[2])
        dqb, _, _ = _bwd_call(qb, kk, vk, sk_b, sk_b, ob, lb, do_b, scale, views[1], views[3])
        dk = torch.empty(B, 2 * n, hkv, d, dtype=do.dtype, device=do.device)
        dv = torch.empty_like(dk)
        native.call("lb_cp_dkv_reduce", ws.arr(ws.grad_off(par, 0)), ws.arr(ws.grad_off(par, 1)), ws.arr(ws.grad_off(par, 2)),
                    ws.arr(ws.grad_off(par, 3)), ws.arr(ws.ready_off), dk.data_ptr(), dv.data_ptr(), B, n, hkv * d, c, r,
                    ws.bwd_calls, native.stream_ptr())
        return torch.cat((dqa, dqb), dim=1), dk, dv, None, None


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
