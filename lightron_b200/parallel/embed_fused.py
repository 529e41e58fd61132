"""Vocab-parallel embedding whose rows travel by peer stores instead of a collective.

The reference's ``VocabParallelEmbedding`` (``parallel/parallel_tp.py:131-143``) masks the ids outside
the local vocab range, looks up a mostly-zero ``[tokens, hidden]`` partial on every rank and
all-reduces it.  Here (``lb_embed_tp_fwd``) the rank that owns a token's id stores that one row
straight into the buffer of the rank that needs it: under sequence parallelism the owner of the
row, otherwise every rank.  Every row crosses NVLink once (n - 1 times when replicated) instead of
the whole partial going through a reduction.  Backward under sequence parallelism
(``lb_embed_tp_bwd``): every rank publishes its gradient rows and adds the rows of the tokens it owns,
read from their owners, into its table gradient; without sequence parallelism the incoming gradient is
already replicated and the local kernel is used.

CPU ranks and groups without peer memory keep the library path of ``parallel/tp.py``.
"""
from __future__ import annotations

import ctypes
from typing import Dict

import torch
import torch.distributed as dist

from ..ops import native

_G = 32


class _Workspace:
    """Two forward and two backward staging buffers (calls alternate: a peer is never more than one
    call ahead, because every call waits for every peer) and one flag table per direction."""

    def __init__(self, group, T: int, H: int, sp: bool, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.key = (T, H, sp)
        self.n, self.rank = dist.get_world_size(group), dist.get_rank(group)
        rows_f = T // self.n if sp else T
        self.fwd_bytes = (rows_f * H * 2 + 255) // 256 * 256
        self.bwd_bytes = ((T // self.n) * H * 2 + 255) // 256 * 256 if sp else 0
        self.flag_bytes = (self.n * _G * 4 + 255) // 256 * 256
        total = 2 * self.flag_bytes + 2 * self.fwd_bytes + 2 * self.bwd_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf[: 2 * self.flag_bytes].zero_()
        hdl = symm_mem.rendezvous(self.buf, group=group)
        off = int(getattr(hdl, "offset", 0))
        self.ptrs = [int(p) + off for p in hdl.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self.calls = [0, 0]

    def arr(self, off: int):
        a = (ctypes.c_void_p * self.n)()
        for r in range(self.n):
            a[r] = self.ptrs[r] + off
        return a

    def stage_off(self, direction: int, parity: int) -> int:
        base = 2 * self.flag_bytes
        return base + parity * self.fwd_bytes if direction == 0 else base + 2 * self.fwd_bytes + parity * self.bwd_bytes


_WS: Dict[int, _Workspace] = {}


def _workspace(group, T, H, sp, device) -> _Workspace:
    ws = _WS.get(id(group))
    if ws is None or ws.key != (T, H, sp):
        if ws is not None:
            torch.cuda.synchronize()
            dist.barrier(group=group)
        ws = _WS[id(group)] = _Workspace(group, T, H, sp, device)
    return ws


def fused_ok(weight: torch.Tensor, group, n_tokens: int, sp: bool) -> bool:
    if not (weight.is_cuda and weight.dtype == torch.bfloat16 and native.available() and weight.shape[1] % 8 == 0):
        return False
    from . import fused, symm
    n = dist.get_world_size(group)
    return fused._FUSED_ENABLED and n > 1 and symm.supported(group) and (not sp or n_tokens % n == 0)


class _PeerEmbedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, weight, group, vocab_start, sp):
        tok = tokens.reshape(-1).contiguous()
        T, H = tok.numel(), weight.shape[1]
        ws = _workspace(group, T, H, sp, weight.device)
        n, me = ws.n, ws.rank
        ws.calls[0] += 1
        out = torch.empty(T // n if sp else T, H, dtype=weight.dtype, device=weight.device)
        native.call("lb_embed_tp_fwd", tok.data_ptr(), weight.data_ptr(), out.data_ptr(),
                    ws.arr(ws.stage_off(0, ws.calls[0] % 2)), ws.arr(0), T, H, vocab_start, vocab_start + weight.shape[0],
                    n, me, _G, int(sp), ws.calls[0], native.stream_ptr())
        ctx.save_for_backward(tok)
        ctx.meta = (group, vocab_start, sp, weight.shape)
        return out

    @staticmethod
    def backward(ctx, dy):
        (tok,) = ctx.saved_tensors
        group, v0, sp, (V, H) = ctx.meta
        dy = dy.contiguous()
        dw = torch.zeros(V, H, dtype=dy.dtype, device=dy.device)
        T = tok.numel()
        if not sp:          # the gradient is already the same on every rank
            native.call("lb_embedding_bwd", tok.data_ptr(), dy.data_ptr(), dw.data_ptr(), T, H, v0, v0 + V, native.stream_ptr())
            return None, dw, None, None, None
        ws = _WS[id(group)]
        ws.calls[1] += 1
        native.call("lb_embed_tp_bwd", tok.data_ptr(), dy.data_ptr(), dw.data_ptr(), ws.arr(ws.stage_off(1, ws.calls[1] % 2)),
                    ws.arr(ws.flag_bytes), T, H, v0, v0 + V, ws.n, ws.rank, _G, ws.calls[1], native.stream_ptr())
        return None, dw, None, None, None


def vocab_parallel_embedding(tokens: torch.Tensor, weight: torch.Tensor, group, vocab_start: int, sp: bool) -> torch.Tensor:
    """tokens [...] (the same on every rank of the group) -> [T, H] rows, or this rank's [T / n, H] rows
    under sequence parallelism.  ``weight`` holds vocab ids [vocab_start, vocab_start + rows)."""
    return _PeerEmbedding.apply(tokens, weight, group, vocab_start, bool(sp))
