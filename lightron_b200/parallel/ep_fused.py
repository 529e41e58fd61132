"""Expert-parallel MoE feed-forward as a chain of sm_100a kernels with no host round trip.

Replaces, for CUDA bf16 runs, what ``parallel/ep.py`` does with library calls (and what the
reference does in ``parallel/parallel_ep.py:7-51,73-182`` and ``model/model.py:96-116``):

=====================  =====================================================================
router                 ``lb_moe_router``: gate GEMM + softmax + top-k + per-block histograms
count exchange / plan  ``lb_moe_plan``: counts stored into every peer's table (flag per source),
                       destination rows, 128-row-aligned expert segments, load-balance loss
dispatch               ``lb_moe_push``: token rows stored straight into the owner's buffer
expert MLPs            ``lb_gemm_ragged`` (waits for the arrival word itself), SwiGLU, ``lb_gemm_ragged``
combine                ``lb_moe_pull``: peer loads + top-k weighted sum + un-permute
=====================  =====================================================================

and the mirror image in backward (``lb_moe_pull`` with dot products for the routed-weight gradients,
``lb_moe_push`` of the scaled output gradient, ragged data / weight gradients, ``lb_moe_pull`` of the
input gradient, ``lb_moe_router_bwd``).  Per-expert token counts exist only in device memory: the
host never waits for them, every tensor on the expert side has the static capacity
``ceil(capacity_factor * tokens * top_k)`` rows (+ padding), and the copies a routing sends beyond it
are dropped (not dispatched, no contribution to the combine), counted in a status word that the
trainer reports (``native.take_moe_dropped``).

With one rank (no expert parallelism) the same kernels run on ordinary device tensors; with several,
the exchange buffers and flag words live in ``torch.distributed._symmetric_memory``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import native

_I32, _F32, _BF16 = torch.int32, torch.float32, torch.bfloat16
_CTRL_BYTES = 8192
_MAX_LOCAL = 8          # local experts per ragged launch (MAX_PROBLEMS of the grouped GEMM)


def _up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def enabled() -> bool:
    return os.environ.get("LIGHTRON_FUSED_EP", "1") != "0"


def supported(x: torch.Tensor, group, num_experts: int, topk: int, local_experts: int) -> bool:
    if not (enabled() and x.is_cuda and x.dtype == _BF16 and native.available()):
        return False
    if x.shape[-1] % 8 or num_experts > 64 or topk > 8 or topk > num_experts or local_experts > _MAX_LOCAL:
        return False
    if group is not None and dist.get_world_size(group) > 1:
        if dist.get_backend(group) != "nccl" or dist.get_world_size(group) > 8:
            return False
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
        except Exception:
            return False
    return True


class Workspace:
    """Exchange buffers and flag words of one expert-parallel group.

    Control page (u32 words unless noted): [0, n) counts arrived; [16] rows arrived in x buffers;
    [17] rows arrived in the dy buffer; [32, 32+n) y ready; [48, 48+n) dx ready;
    [1024, 1024 + 2*n*E) int32 count tables.  Data: per MoE layer an x buffer and a y buffer (both kept
    until the layer's backward), plus one dy and one dx buffer shared by all layers (a rank can
    only reach layer L-1's backward exchange after every rank has finished layer L's).
    """

    def __init__(self, group, n: int, rank: int, H: int, cap: int, E: int, device):
        self.group, self.n, self.rank, self.H, self.cap, self.E = group, n, rank, H, cap, E
        self.device = device
        self.buf_bytes = _up(cap * H * 2, 4096)
        self.layers: Dict[int, int] = {}          # layer key -> slot
        self.slots: List[dict] = []
        self.epoch_cnt = 0
        self.arr_x = 0
        self.arr_dy = 0
        self.epoch_y = 0
        self.epoch_dx = 0
        self.ctrl, self.ctrl_ptrs = self._alloc(_CTRL_BYTES, zero=True)
        self.dy, self.dy_ptrs = self._alloc(self.buf_bytes)
        self.dx, self.dx_ptrs = self._alloc(self.buf_bytes)

    def _alloc(self, nbytes: int, zero: bool = False):
        if self.n == 1:
            t = torch.zeros(nbytes, dtype=torch.uint8, device=self.device) if zero else \
                torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            return t, [t.data_ptr()]
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        if zero:
            t.zero_()
        hdl = symm_mem.rendezvous(t, group=self.group)
        off = int(getattr(hdl, "offset", 0))
        ptrs = [int(p) + off for p in hdl.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier(group=self.group)           # zeroed everywhere before anybody's first store
        return t, ptrs

    def slot(self, key: int) -> dict:
        """The (x, y) buffers of MoE layer `key`; allocated collectively at its first forward."""
        if key not in self.layers:
            x, xp = self._alloc(self.buf_bytes)
            y, yp = self._alloc(self.buf_bytes)
            self.layers[key] = len(self.slots)
            self.slots.append({"x": x, "x_ptrs": xp, "y": y, "y_ptrs": yp})
        return self.slots[self.layers[key]]

    def view(self, buf: torch.Tensor) -> torch.Tensor:
        return buf[: self.cap * self.H * 2].view(_BF16).view(self.cap, self.H)

    def ptrs(self, base: Sequence[int], off: int = 0):
        arr = (ctypes.c_void_p * self.n)()
        for r in range(self.n):
            arr[r] = base[r] + off
        return arr


_WS: Dict[tuple, Workspace] = {}


def workspace(group, H: int, cap: int, E: int, device) -> Workspace:
    n = dist.get_world_size(group) if group is not None else 1
    rank = dist.get_rank(group) if group is not None else 0
    key = (id(group), H, cap, E)
    ws = _WS.get(key)
    if ws is None:
        ws = _WS[key] = Workspace(group, n, rank, H, cap, E, device)
    return ws


def _ptr_array(tensors: Sequence[torch.Tensor]):
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


def _ragged(A, B_list, C, seg, LE, cap, N, K, b_mn, wait_flag=0, wait_target=0):
    ldb = B_list[0].stride(0)
    native.call("lb_gemm_ragged", A.data_ptr(), _ptr_array(B_list), C.data_ptr(), seg.data_ptr(), LE, cap, N, K,
                A.stride(0), ldb, C.stride(0), int(b_mn), wait_flag, wait_target, native.stream_ptr())


def _ragged_wgrad(dY, X, C_list, seg, LE, cap, Nw, Kw):
    native.call("lb_gemm_ragged_wgrad", dY.data_ptr(), X.data_ptr(), _ptr_array(C_list), seg.data_ptr(), LE, cap, Nw, Kw,
                dY.stride(0), X.stride(0), C_list[0].stride(0), 1, native.stream_ptr())


class _FusedMoE(torch.autograd.Function):
    """x [T, H], gate weight [E, H], then per local expert its (w1, w3, w2) -> (out [T, H], aux [1])."""

    @staticmethod
    def forward(ctx, x, gate_w, meta, *expert_ws):
        ws: Workspace = meta["ws"]
        E, k, LE, cap, n, me = meta["E"], meta["k"], meta["LE"], ws.cap, ws.n, ws.rank
        T, H = x.shape
        I = expert_ws[0].shape[0]
        dev = x.device
        x = x.contiguous()
        st = native.stream_ptr
        nblk = native.require().lb_moe_router_blocks(T)
        probs = torch.empty(T, E, dtype=_F32, device=dev)
        idx = torch.empty(T, k, dtype=_I32, device=dev)
        wts = torch.empty(T, k, dtype=_F32, device=dev)
        within = torch.zeros(nblk * 32, k, dtype=_I32, device=dev)
        blk_hist = torch.empty(nblk, E, dtype=_I32, device=dev)
        blk_psum = torch.empty(nblk, E, dtype=_F32, device=dev)
        native.call("lb_moe_router", x.data_ptr(), gate_w.data_ptr(), T, H, E, k, probs.data_ptr(), idx.data_ptr(),
                    wts.data_ptr(), within.data_ptr(), blk_hist.data_ptr(), blk_psum.data_ptr(), st())
        blk_base = torch.empty(nblk, E, dtype=_I32, device=dev)
        dst_row0 = torch.empty(E, dtype=_I32, device=dev)
        seg = torch.zeros(2 * LE + 2, dtype=_I32, device=dev)
        frac = torch.empty(E, dtype=_F32, device=dev)
        aux = torch.empty(1, dtype=_F32, device=dev)
        ws.epoch_cnt += 1
        native.call("lb_moe_plan", blk_hist.data_ptr(), blk_psum.data_ptr(), blk_base.data_ptr(), dst_row0.data_ptr(),
                    seg.data_ptr(), frac.data_ptr(), aux.data_ptr(), nblk, E, n, me, T, k, cap,
                    ws.ptrs(ws.ctrl_ptrs, 4096), ws.ptrs(ws.ctrl_ptrs, 0), ws.epoch_cnt & 1, ws.epoch_cnt, st())
        slot = ws.slot(meta["layer_key"])
        rows = torch.empty(T, k, dtype=_I32, device=dev)
        G = native.require().lb_moe_push_ctas(T)
        ws.arr_x += n * G
        native.call("lb_moe_push", x.data_ptr(), 0, idx.data_ptr(), within.data_ptr(), blk_base.data_ptr(),
                    dst_row0.data_ptr(), rows.data_ptr(), seg.data_ptr(), T, H, E, k, n, me, cap, 1,
                    ws.ptrs(slot["x_ptrs"]), ws.ptrs(ws.ctrl_ptrs, 64), st())
        xbuf, ybuf = ws.view(slot["x"]), ws.view(slot["y"])
        ups = [OF._as_strided_cat(expert_ws[3 * e:3 * e + 2]) for e in range(LE)]       # [2I, H] gate | up
        downs = [expert_ws[3 * e + 2] for e in range(LE)]                               # [H, I]
        gu = torch.empty(cap, 2 * I, dtype=_BF16, device=dev)
        _ragged(xbuf, ups, gu, seg, LE, cap, 2 * I, H, False, ws.ctrl_ptrs[me] + 64, ws.arr_x)
        a = torch.empty(cap, I, dtype=_BF16, device=dev)
        rows_dev = seg.data_ptr() + 4 * (2 * LE)                                          # padded end of the last segment
        native.call("lb_swiglu_fwd_dev", gu.data_ptr(), a.data_ptr(), cap, I, gu.stride(0), rows_dev, st())
        _ragged(a, downs, ybuf, seg, LE, cap, H, I, False)
        out = torch.empty(T, H, dtype=_BF16, device=dev)
        ws.epoch_y += 1
        native.call("lb_moe_pull", out.data_ptr(), wts.data_ptr(), idx.data_ptr(), rows.data_ptr(), 0, 0, T, H, E, k, n,
                    me, cap, ws.ptrs(slot["y_ptrs"]), ws.ptrs(ws.ctrl_ptrs, 128), ws.epoch_y, st())
        ctx.save_for_backward(x, gate_w, probs, idx, wts, rows, seg, frac, gu, a, *expert_ws)
        ctx.meta, ctx.slot, ctx.params = meta, slot, expert_ws
        return out, aux

    @staticmethod
    def backward(ctx, dout, daux):
        x, gate_w, probs, idx, wts, rows, seg, frac, gu, a, *expert_ws = ctx.saved_tensors
        meta, slot = ctx.meta, ctx.slot
        ws: Workspace = meta["ws"]
        E, k, LE, cap, n, me = meta["E"], meta["k"], meta["LE"], ws.cap, ws.n, ws.rank
        T, H = x.shape
        I = expert_ws[0].shape[0]
        dev = x.device
        st = native.stream_ptr
        dout = dout.contiguous()
        xbuf, ybuf = ws.view(slot["x"]), ws.view(slot["y"])
        dybuf, dxbuf = ws.view(ws.dy), ws.view(ws.dx)
        # routed-weight gradients: <dout[t], y[row(t, s)]>, read from the owners once more
        dwts = torch.empty(T, k, dtype=_F32, device=dev)
        ws.epoch_y += 1
        native.call("lb_moe_pull", 0, 0, idx.data_ptr(), rows.data_ptr(), dwts.data_ptr(), dout.data_ptr(), T, H, E, k, n,
                    me, cap, ws.ptrs(slot["y_ptrs"]), ws.ptrs(ws.ctrl_ptrs, 128), ws.epoch_y, st())
        # dy[row] = w[t, s] * dout[t], stored into the owners' dy buffers
        G = native.require().lb_moe_push_ctas(T)
        ws.arr_dy += n * G
        native.call("lb_moe_push", dout.data_ptr(), wts.data_ptr(), idx.data_ptr(), 0, 0, 0, rows.data_ptr(), seg.data_ptr(),
                    T, H, E, k, n, me, cap, 0, ws.ptrs(ws.dy_ptrs), ws.ptrs(ws.ctrl_ptrs, 68), st())
        params = ctx.params
        direct = all(getattr(w, "_lb_direct_grad", False) and w.grad is not None for w in params) and \
            all(OF._rows_adjacent([params[3 * e].grad, params[3 * e + 1].grad]) for e in range(LE))
        if direct:
            g_up = [OF._as_strided_cat([params[3 * e].grad, params[3 * e + 1].grad]) for e in range(LE)]
            g_down = [params[3 * e + 2].grad for e in range(LE)]
        else:
            g_up = [torch.zeros(2 * I, H, dtype=_BF16, device=dev) for _ in range(LE)]
            g_down = [torch.zeros(H, I, dtype=_BF16, device=dev) for _ in range(LE)]
        ups = [OF._as_strided_cat(expert_ws[3 * e:3 * e + 2]) for e in range(LE)]
        downs = [expert_ws[3 * e + 2] for e in range(LE)]
        # down projection: da = dy W2, dW2 += dy^T a
        da = torch.empty(cap, I, dtype=_BF16, device=dev)
        _ragged(dybuf, downs, da, seg, LE, cap, I, H, True, ws.ctrl_ptrs[me] + 68, ws.arr_dy)
        _ragged_wgrad(dybuf, a, g_down, seg, LE, cap, H, I)
        dgu = torch.empty(cap, 2 * I, dtype=_BF16, device=dev)
        rows_dev = seg.data_ptr() + 4 * (2 * LE)
        native.call("lb_swiglu_bwd_dev", gu.data_ptr(), da.data_ptr(), dgu.data_ptr(), cap, I, gu.stride(0), rows_dev, st())
        # gate | up projection: dx_rows = dgu [W1; W3], d[W1; W3] += dgu^T x_rows
        _ragged(dgu, ups, dxbuf, seg, LE, cap, H, 2 * I, True)
        _ragged_wgrad(dgu, xbuf, g_up, seg, LE, cap, 2 * I, H)
        # input gradient: sum of the k rows, read from their owners
        dx = torch.empty(T, H, dtype=_BF16, device=dev)
        ws.epoch_dx += 1
        native.call("lb_moe_pull", dx.data_ptr(), 0, idx.data_ptr(), rows.data_ptr(), 0, 0, T, H, E, k, n, me, cap,
                    ws.ptrs(ws.dx_ptrs), ws.ptrs(ws.ctrl_ptrs, 192), ws.epoch_dx, st())
        # router
        dx_r = torch.empty(T, H, dtype=_BF16, device=dev)
        dwg = torch.zeros(E, H, dtype=_F32, device=dev)
        daux_ptr = 0
        if daux is not None:
            daux = daux.to(_F32).contiguous()
            daux_ptr = daux.data_ptr()
        native.call("lb_moe_router_bwd", x.data_ptr(), gate_w.data_ptr(), probs.data_ptr(), idx.data_ptr(), dwts.data_ptr(),
                    frac.data_ptr(), daux_ptr, dx_r.data_ptr(), dwg.data_ptr(), T, H, E, k, st())
        native.call("lb_add_inplace", dx.data_ptr(), dx_r.data_ptr(), dx.numel(), st())
        if direct:
            for w in params:
                for hook in getattr(w, "_lb_grad_hooks", ()):
                    hook(w)
            egrads = [None] * len(params)
        else:
            egrads = []
            for e in range(LE):
                egrads += [g_up[e][:I], g_up[e][I:], g_down[e]]
        return (dx, dwg.to(gate_w.dtype), None, *egrads)


def fused_moe(x: torch.Tensor, gate_w: torch.Tensor, expert_ws: Sequence[torch.Tensor], num_experts: int, topk: int,
              group, layer_key: int, capacity_factor: float = 2.0):
    """x [T, H] -> (out [T, H], aux loss [1]).  expert_ws: (w1, w3, w2) of every local expert, in
    expert order, w1 and w3 row-adjacent in memory (they are in the flat parameter arena)."""
    T, H = x.shape
    n = dist.get_world_size(group) if group is not None else 1
    LE = num_experts // n
    if n == 1 and capacity_factor >= 1.0:
        cap = _up(T * topk, 128) + LE * 128          # one rank can never receive more than its own copies
    else:
        cap = _up(int(capacity_factor * T * topk), 128) + LE * 128
    ws = workspace(group, H, cap, num_experts, x.device)
    meta = {"ws": ws, "E": num_experts, "k": topk, "LE": LE, "layer_key": layer_key}
    return _FusedMoE.apply(x, gate_w, meta, *expert_ws)
