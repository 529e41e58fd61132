"""Peer-memory workspace and the fused compute + collective ops of sequence-parallel TP.

``AllGatherLinear``       all-gather(rows) -> GEMM      one kernel (``lb_gemm_ag``)
``LinearReduceScatter``   GEMM -> reduce-scatter(rows)  one kernel (``lb_gemm_rs``)

The NVLink plumbing: one symmetric allocation per tensor-parallel group
(``torch.distributed._symmetric_memory``: every rank maps every peer's buffer), holding
 * block counters (32-bit words, zeroed once, then only ever growing: every call knows the value
   that means "this call's data has arrived", so nothing is ever reset),
 * a ring of gather buffers ``[tokens, width]`` that peers PUSH their rows into.  Forward gathers
   are kept for backward (wgrad needs the gathered operand), so the ring holds two micro-batch
   generations of forward calls: a buffer is rewritten only after every rank has gone through a
   whole further forward + backward, i.e. long after its last reader.  With 180 GB per GPU this
   costs a few GB and removes both the re-gather and any copy out of peer-visible memory;
 * a 2-deep ring of gather buffers for backward-only gathers and a 2-deep ring of
   reduce-scatter receive areas.  Two are enough without acknowledgements: a rank can only
   start call c+2 after every peer has entered call c+1 (it needs their data), i.e. after they
   finished reading call c.

The kernels write peers with plain coalesced stores (stores are fire-and-forget, so a few CTAs
fill NVLink) and read only local memory; no TMA multicast, no library kernel is ever handed a
peer pointer.  Every wait on a peer's counter is bounded in the kernel and reports through
``lb_device_status``.

Reference counterparts: ``funcol.all_gather_tensor`` + ``F.linear`` and ``F.linear`` +
``funcol.reduce_scatter_tensor`` (parallel/parallel_tp.py:61-69, 100-106).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import native

_BM = 128
_MAX_BLOCKS = 4096             # 128-row blocks per gather buffer (tokens <= 524288)
_MAX_BPR = 1024
_MOVER_WARPS = 6               # warps per mover CTA: each adds 1 to a block counter
N_COMM_CTAS = int(os.environ.get("LIGHTRON_AG_CTAS", "0"))     # 0 = choose per call from the GEMM size
# how the gathered rows travel: "sm" = mover CTAs inside the GEMM kernel (peer stores), "ce" = copy-engine
# transfers issued next to the kernel (about twice the link rate; the kernel consumes blocks as they land)
AG_TRANSPORT = os.environ.get("LIGHTRON_AG_TRANSPORT", "sm")
DEFAULT_KEEP_SLOTS = 8


def _up(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class Workspace:
    """Symmetric buffer layout (bytes):
    [ag counters: (keep + 2) x MAX_BLOCKS u32][rs counters: 2 x 8 x MAX_BPR u32]
    [keep gather ring][2 scratch gather buffers][2 receive areas]"""

    def __init__(self, group, gather_bytes: int, recv_bytes: int, keep_slots: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.n = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.gather_bytes = _up(gather_bytes)
        self.recv_bytes = _up(recv_bytes)
        self.keep_slots = keep_slots
        self.n_gather = keep_slots + 2
        self.ag_flag_off = 0
        self.rs_flag_off = _up(self.n_gather * _MAX_BLOCKS * 4)
        self.data_off = _up(self.rs_flag_off + 2 * 8 * _MAX_BPR * 4, 4096)
        self.recv_off0 = self.data_off + self.n_gather * self.gather_bytes
        total = self.recv_off0 + 2 * self.recv_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf[: self.data_off].zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group=group)
        off = int(getattr(self.hdl, "offset", 0))          # the tensor may sit inside a larger symmetric block
        self.ptrs: List[int] = [int(p) + off for p in self.hdl.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier(group=group)            # everybody's counters are zero before anybody pushes
        self.keep_calls = 0
        self.scratch_calls = 0
        self.rs_calls = 0
        self.ag_uses = [0] * self.n_gather   # how often each gather buffer has been a destination
        self.generation = [0] * self.n_gather
        self.rs_target = [0, 0]
        self.ag_blocks = [None] * self.n_gather   # row blocks of the last gather into each buffer
        self.rs_bpr = [None, None]                # row blocks per rank of the last reduce-scatter per receive area

    def resync(self) -> None:
        """Collective: zero every counter.  The counters of a buffer grow by a fixed amount per use, per
        128-row block; when a call uses a buffer with another number of blocks than the call before
        (a different token count: rare, e.g. an evaluation batch) the blocks would disagree about the
        target, so all ranks drain their streams, zero their counters and start counting afresh."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)            # nobody is still adding to anybody's counters
        self.buf[: self.data_off].zero_()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self.ag_uses = [0] * self.n_gather
        self.rs_target = [0, 0]
        self.ag_blocks = [None] * self.n_gather
        self.rs_bpr = [None, None]

    def gather_off(self, slot: int) -> int:
        return self.data_off + slot * self.gather_bytes

    def recv_off(self, slot: int) -> int:
        return self.recv_off0 + slot * self.recv_bytes

    def local_view(self, off: int, rows: int, cols: int) -> torch.Tensor:
        return self.buf[off:off + rows * cols * 2].view(torch.bfloat16).view(rows, cols)

    def ptr_array(self, off: int):
        arr = (ctypes.c_void_p * self.n)()
        for r in range(self.n):
            arr[r] = self.ptrs[r] + off
        return arr

    def next_gather_slot(self, keep: bool, blocks: int) -> int:
        if keep:
            slot = self.keep_calls % self.keep_slots
            self.keep_calls += 1
        else:
            slot = self.keep_slots + self.scratch_calls % 2
            self.scratch_calls += 1
        if self.ag_blocks[slot] not in (None, blocks):
            self.resync()
        self.ag_blocks[slot] = blocks
        self.ag_uses[slot] += 1
        self.generation[slot] += 1
        return slot


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
    return rows_total % (_BM * n) == 0 and rows_total // _BM <= _MAX_BLOCKS and rows_total // n // _BM <= _MAX_BPR


def workspace(group, gather_bytes: int, recv_bytes: int, device, keep_slots: int = 0) -> Workspace:
    """The group's workspace, (re)created collectively when a larger one is needed."""
    ws = _WS.get(id(group))
    if ws is None or ws.gather_bytes < gather_bytes or ws.recv_bytes < recv_bytes or ws.keep_slots < keep_slots:
        if ws is not None:
            torch.cuda.synchronize()
            dist.barrier(group=group)
            gather_bytes, recv_bytes = max(gather_bytes, ws.gather_bytes), max(recv_bytes, ws.recv_bytes)
            keep_slots = max(keep_slots, ws.keep_slots)
        ws = _WS[id(group)] = Workspace(group, gather_bytes, recv_bytes, max(keep_slots, DEFAULT_KEEP_SLOTS), device)
    return ws


def presize(group, tokens: int, width: int, device, fwd_gathers_in_flight: int = 4) -> None:
    """Create the workspace once: [tokens, width] activations, and a keep ring of twice the number
    of forward gathers that can be alive between a forward and its backward."""
    workspace(group, tokens * width * 2, tokens * width * 2, device, keep_slots=2 * fwd_gathers_in_flight)


def check_status() -> None:
    """Raise if a bounded device-side wait ran out since the last check (synchronises)."""
    buf = (ctypes.c_uint * 4)()
    native.require().lb_device_status(ctypes.cast(buf, ctypes.c_void_p))
    if buf[0]:
        raise RuntimeError(f"fused comm kernel gave up waiting (code {buf[0]}, where {buf[1]}): a peer did not arrive")
    native.require().lb_gemm_grouped_status(ctypes.cast(buf, ctypes.c_void_p))
    if buf[0]:
        raise RuntimeError(f"grouped GEMM kernel gave up waiting (code {buf[0]}, where {buf[1]})")


# ---- raw ops ------------------------------------------------------------------------------------------


def ag_gemm(x_local: torch.Tensor, w: torch.Tensor, group, b_mn: bool = False, keep: bool = False):
    """x_local [M/n, K] (this rank's rows), w [N, K] (or [K, N] with b_mn) ->
    (y [M, N] = gather(x) op(w)^T, gathered [M, K], (slot, generation)).
    ``gathered`` is a view of the workspace: with ``keep`` it stays valid for two micro-batch
    generations of forward gathers, otherwise until the call after the next."""
    n = dist.get_world_size(group)
    rows, K = x_local.shape
    M = rows * n
    N = w.shape[1] if b_mn else w.shape[0]
    ws = workspace(group, M * K * 2, 0, x_local.device)
    slot = ws.next_gather_slot(keep, M // _BM)
    target = ws.ag_uses[slot] * _MOVER_WARPS
    y = torch.empty(M, N, dtype=x_local.dtype, device=x_local.device)
    # CTAs that push rows instead of doing MMAs: a short GEMM needs the gather done quickly (more
    # movers), a long one hides it behind the math anyway (fewer movers, more tensor-core SMs).
    n_comm = N_COMM_CTAS
    if AG_TRANSPORT == "ce":
        n_comm = -1                 # copy-engine transfers on a side stream, all SMs on the GEMM
    elif n_comm <= 0:
        flops = 2.0 * M * N * K
        n_comm = 32 if flops < 1.2e11 else (16 if flops < 6e11 else 8)
    gathers = ws.ptr_array(ws.gather_off(slot))
    flags = ws.ptr_array(ws.ag_flag_off + slot * _MAX_BLOCKS * 4)
    native.call("lb_gemm_ag", w.data_ptr(), y.data_ptr(), M, N, K, w.stride(0), y.stride(0), int(b_mn), n, ws.rank,
                x_local.data_ptr(), x_local.stride(0), gathers, flags, target, n_comm, native.stream_ptr())
    gathered = ws.local_view(ws.gather_off(slot), M, K)
    return y, gathered, (slot, ws.generation[slot])


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
    assert bpr <= _MAX_BPR
    if ws.rs_bpr[slot] not in (None, bpr):
        ws.resync()
    ws.rs_bpr[slot] = bpr
    ws.rs_target[slot] += 4 * ((N + 255) // 256)
    out = torch.empty(M // n, N, dtype=x.dtype, device=x.device)
    recv = ws.ptr_array(ws.recv_off(slot))
    flags = ws.ptr_array(ws.rs_flag_off + slot * 8 * _MAX_BPR * 4)
    native.call("lb_gemm_rs", x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0), w.stride(0), int(b_mn), n, ws.rank,
                recv, flags, ws.rs_target[slot], out.data_ptr(), out.stride(0), native.stream_ptr())
    return out


# ---- autograd -------------------------------------------------------------------------------------------


_SCRATCH_TAG = "symm-scratch-gather"


class AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, group, *ws):
        fused = OF._rows_adjacent(ws)
        x_local = x_local.contiguous()
        if fused:
            y, gathered, tag = ag_gemm(x_local, OF._as_strided_cat(ws), group, keep=True)
        else:
            y0, gathered, tag = ag_gemm(x_local, ws[0], group, keep=True)
            y = torch.cat([y0] + [OF.gemm(gathered, w) for w in ws[1:]], dim=1)
        ctx.save_for_backward(*ws)
        ctx.params = ws
        ctx.gathered, ctx.tag = gathered, tag
        ctx.group, ctx.fused = group, fused
        return y

    @staticmethod
    def backward(ctx, dy):
        ws = ctx.saved_tensors
        gathered, (slot, gen) = ctx.gathered, ctx.tag
        wsp = _WS[id(ctx.group)]
        if wsp.generation[slot] != gen:
            raise RuntimeError("gathered activation was overwritten before its backward: the keep ring of the "
                               "peer-memory workspace is too small (symm.presize(..., fwd_gathers_in_flight=...))")
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
        if OF._DEFER_WGRAD and ctx.fused and all(ctx.needs_input_grad[2:]) and OF.direct_wgrad_ok(ctx.params):
            # queued: launched together with the neighbouring layers' weight gradients.  The gathered
            # activation sits in the keep ring, which nobody overwrites before the next forward.
            OF.defer_wgrad(dy, gathered, ctx.params)
            return (dx, None, *([None] * len(ws)))
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
        ctx.params = (w,)
        ctx.group = group
        return gemm_rs(x, w, group)

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        # A queued weight gradient that reads a scratch gather buffer must be launched before this
        # rank's next scratch gather: until then no peer can have reached the call that recycles it.
        if OF.wgrad_queue_uses(_SCRATCH_TAG):
            OF.flush_wgrads(final=False)
        dx, dy_full, _ = ag_gemm(dy_local.contiguous(), w, ctx.group, b_mn=True, keep=False)
        if OF._DEFER_WGRAD and ctx.needs_input_grad[1] and OF.direct_wgrad_ok(ctx.params):
            OF.defer_wgrad(dy_full, x, ctx.params, tag=_SCRATCH_TAG)
            return dx, None, None
        dw = OF.gemm(dy_full, x, a_mn=True, b_mn=True)
        return dx, dw, None
