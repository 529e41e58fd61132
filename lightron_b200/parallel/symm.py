"""Peer-memory workspace and the fused compute + collective ops of sequence-parallel TP.

``AllGatherLinear``       all-gather(rows) -> GEMM      one kernel (``lb_gemm_ag``)
``LinearReduceScatter``   GEMM -> reduce-scatter(rows)  one kernel (``lb_gemm_rs``)

The NVLink plumbing: one symmetric allocation per tensor-parallel group
(``torch.distributed._symmetric_memory``: every rank maps every peer's buffer), holding
 * ready flags and reduce-scatter counters (32-bit words, zeroed once, then only ever growing:
   every call knows the value that means "this call's data", so nothing is reset), and
 * two slots each for all-gather sources and reduce-scatter receive areas.  Two slots are enough
   without acknowledgements: a rank can only start call c+1 after every peer has entered call c+1
   (it needs their data), i.e. after they finished reading / reducing call c.

The kernels read peers with plain loads and write peers with plain stores from the GEMM
epilogue; no TMA multicast, no library kernel is ever handed a peer pointer.  Every wait on a
peer's flag is bounded in the kernel and reports through ``lb_device_status``.

Reference counterparts: ``funcol.all_gather_tensor`` + ``F.linear`` and ``F.linear`` +
``funcol.reduce_scatter_tensor`` (parallel/parallel_tp.py:61-69, 100-106).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import native

_BM = 128
_FLAG_BYTES = 128 * 1024
_READY_OFF = 0                 # [2 slots][8 ranks] u32
_RS_OFF = 256                  # [2 slots][n][blocks_per_rank] u32
_MAX_BPR = 1024
N_COMM_CTAS = int(os.environ.get("LIGHTRON_AG_CTAS", "16"))


class Workspace:
    def __init__(self, group, src_bytes: int, recv_bytes: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.n = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.src_bytes = (src_bytes + 255) // 256 * 256
        self.recv_bytes = (recv_bytes + 255) // 256 * 256
        total = _FLAG_BYTES + 2 * self.src_bytes + 2 * self.recv_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group=group)
        self.ptrs: List[int] = [int(p) for p in self.hdl.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier(group=group)            # everybody's flags are zero before anybody signals
        self.block_flags = torch.zeros(2, 4 * _MAX_BPR, dtype=torch.int32, device=device)   # local only
        self.ag_calls = 0
        self.rs_calls = 0
        self.rs_target = [0, 0]

    def src_off(self, slot: int) -> int:
        return _FLAG_BYTES + slot * self.src_bytes

    def recv_off(self, slot: int) -> int:
        return _FLAG_BYTES + 2 * self.src_bytes + slot * self.recv_bytes

    def local_view(self, off: int, rows: int, cols: int) -> torch.Tensor:
        return self.buf[off:off + rows * cols * 2].view(torch.bfloat16).view(rows, cols)

    def ptr_array(self, off: int):
        arr = (ctypes.c_void_p * self.n)()
        for r in range(self.n):
            arr[r] = self.ptrs[r] + off
        return arr


_WS: Dict[int, Workspace] = {}
_SUPPORT: Dict[int, bool] = {}


def supported(group) -> bool:
    if os.environ.get("LIGHTRON_FUSED_COMM", "1") == "0":
        return False
    key = id(group)
    if key not in _SUPPORT:
        ok = native.available() and dist.get_backend(group) == "nccl" and dist.get_world_size(group) <= 8
        if ok:
            try:
                import torch.distributed._symmetric_memory  # noqa: F401
            except Exception:
                ok = False
        _SUPPORT[key] = ok
    return _SUPPORT[key]


def shapes_ok(rows_total: int, group) -> bool:
    n = dist.get_world_size(group)
    return rows_total % (_BM * n) == 0 and rows_total // n // _BM <= _MAX_BPR


def workspace(group, src_bytes: int, recv_bytes: int, device) -> Workspace:
    ws = _WS.get(id(group))
    if ws is None or ws.src_bytes < src_bytes or ws.recv_bytes < recv_bytes:
        if ws is not None:
            torch.cuda.synchronize()
            dist.barrier(group=group)
            src_bytes, recv_bytes = max(src_bytes, ws.src_bytes), max(recv_bytes, ws.recv_bytes)
        ws = _WS[id(group)] = Workspace(group, src_bytes, recv_bytes, device)
    return ws


def presize(group, tokens: int, width: int, device) -> None:
    """Create the workspace once with room for [tokens, width] activations (avoids regrowth)."""
    n = dist.get_world_size(group)
    workspace(group, (tokens // n) * width * 2, tokens * width * 2, device)


def check_status() -> None:
    """Raise if a bounded device-side wait ran out since the last check (synchronises)."""
    buf = (ctypes.c_uint * 4)()
    native.require().lb_device_status(ctypes.cast(buf, ctypes.c_void_p))
    if buf[0]:
        raise RuntimeError(f"fused comm kernel gave up waiting (code {buf[0]}, where {buf[1]}): a peer did not arrive")


# ---- raw ops ------------------------------------------------------------------------------------------


def ag_gemm(x_local: torch.Tensor, w: torch.Tensor, group, b_mn: bool = False):
    """x_local [M/n, K] (this rank's rows), w [N, K] (or [K, N] with b_mn) ->
    (y [M, N] = gather(x) op(w)^T, gathered [M, K])."""
    n = dist.get_world_size(group)
    rows, K = x_local.shape
    M = rows * n
    N = w.shape[1] if b_mn else w.shape[0]
    ws = workspace(group, rows * K * 2, 0, x_local.device)
    slot = ws.ag_calls % 2
    epoch = ws.ag_calls // 2 + 1
    ws.ag_calls += 1
    src = ws.local_view(ws.src_off(slot), rows, K)
    src.copy_(x_local)                               # stage this rank's rows where peers can read them
    gathered = torch.empty(M, K, dtype=x_local.dtype, device=x_local.device)
    y = torch.empty(M, N, dtype=x_local.dtype, device=x_local.device)
    ready = ws.ptr_array(_READY_OFF + slot * 8 * 4)
    srcs = ws.ptr_array(ws.src_off(slot))
    native.call("lb_gemm_ag", w.data_ptr(), y.data_ptr(), M, N, K, w.stride(0), y.stride(0), int(b_mn), n, ws.rank,
                srcs, K, gathered.data_ptr(), ready, ws.block_flags[slot].data_ptr(), epoch, N_COMM_CTAS,
                native.stream_ptr())
    return y, gathered


def gemm_rs(x: torch.Tensor, w: torch.Tensor, group, b_mn: bool = False) -> torch.Tensor:
    """x [M, K_local], w [N, K_local] (or [K_local, N] with b_mn) -> this rank's [M/n, N] rows of
    sum_over_ranks(x op(w)^T)."""
    n = dist.get_world_size(group)
    M, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    ws = workspace(group, 0, M * N * 2, x.device)
    slot = ws.rs_calls % 2
    ws.rs_calls += 1
    bpr = M // n // _BM
    ws.rs_target[slot] += 4 * ((N + 255) // 256)
    out = torch.empty(M // n, N, dtype=x.dtype, device=x.device)
    recv = ws.ptr_array(ws.recv_off(slot))
    flags = ws.ptr_array(_RS_OFF + slot * 8 * _MAX_BPR * 4)
    assert bpr <= _MAX_BPR
    native.call("lb_gemm_rs", x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0), w.stride(0), int(b_mn), n, ws.rank,
                recv, flags, ws.rs_target[slot], out.data_ptr(), out.stride(0), native.stream_ptr())
    return out


# ---- autograd -------------------------------------------------------------------------------------------


class AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, group, *ws):
        fused = OF._rows_adjacent(ws)
        wcat = OF._as_strided_cat(ws) if fused else None
        if fused:
            y, gathered = ag_gemm(x_local.contiguous(), wcat, group)
        else:
            y0, gathered = ag_gemm(x_local.contiguous(), ws[0], group)
            y = torch.cat([y0] + [OF.gemm(gathered, w) for w in ws[1:]], dim=1)
        ctx.save_for_backward(gathered, *ws)
        ctx.group, ctx.fused = group, fused
        return y

    @staticmethod
    def backward(ctx, dy):
        gathered, *ws = ctx.saved_tensors
        dy = dy.contiguous()
        sizes = [w.shape[0] for w in ws]
        if ctx.fused:
            dx = gemm_rs(dy, OF._as_strided_cat(ws), ctx.group, b_mn=True)
        else:
            full, off = None, 0
            for w, nn_ in zip(ws, sizes):
                part = OF.gemm(dy[:, off:off + nn_], w, b_mn=True)
                full = part if full is None else full.add_(part)
                off += nn_
            from . import comm
            dx = comm.reduce_scatter_rows(full, ctx.group)
        dw = OF.gemm(dy, gathered, a_mn=True, b_mn=True)
        dws, off = [], 0
        for nn_ in sizes:
            dws.append(dw[off:off + nn_])
            off += nn_
        return (dx, None, *dws)


class LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group):
        x = x.contiguous()
        ctx.save_for_backward(x, w)
        ctx.group = group
        return gemm_rs(x, w, group)

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        dx, dy_full = ag_gemm(dy_local.contiguous(), w, ctx.group, b_mn=True)
        dw = OF.gemm(dy_full, x, a_mn=True, b_mn=True)
        return dx, dw, None
