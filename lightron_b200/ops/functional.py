"""Differentiable ops.  CUDA bf16 tensors run the hand-written sm_100a kernels; every other
tensor runs the PyTorch oracle in ``ops.reference`` (CPU ranks, fp32 parity runs).

Call sites these replace in the reference: ``F.linear`` (parallel/parallel_tp.py:69,100;
model/model.py:155,202), ``RMSNorm`` (layers/layers.py:5-16), ``apply_rotary_emb``
(layers/layers.py:44-70), ``F.silu(w1 x) * w3 x`` (model/model.py:69),
``F.scaled_dot_product_attention`` (model/model.py:193-198), ``F.embedding`` (model/model.py:261)
and ``F.cross_entropy`` (trainer.py:52).
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import native, reference as ref

# --------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------


def _rows_adjacent(ws: Sequence[torch.Tensor]) -> bool:
    """True when the [n_i, K] matrices sit back to back in memory (one [sum n_i, K] matrix)."""
    for a, b in zip(ws[:-1], ws[1:]):
        if not (a.is_contiguous() and b.is_contiguous()):
            return False
        if a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr():
            return False        # neighbours by accident of the allocator, not one buffer
        if a.data_ptr() + a.numel() * a.element_size() != b.data_ptr():
            return False
    return True


def _as_strided_cat(ws: Sequence[torch.Tensor]) -> torch.Tensor:
    """View adjacent [n_i, K] matrices as one [sum n_i, K] matrix without copying."""
    n = sum(w.shape[0] for w in ws)
    return ws[0].as_strided((n, ws[0].shape[1]), (ws[0].shape[1], 1))


def gemm(a: torch.Tensor, b: torch.Tensor, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, legacy: bool = False) -> torch.Tensor:
    """C[M,N] = A . B^T on the tcgen05 kernel.  ``a_mn``: A is stored [K, M] (M contiguous)
    instead of [M, K]; ``b_mn``: B is stored [K, N] instead of [N, K].  Row strides are free
    (multiples of 8 elements), inner stride must be 1."""
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert K == Kb, f"K mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, dtype=a.dtype, device=a.device)
    native.call("lb_gemm_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
                a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn), int(legacy), native.stream_ptr())
    return out


def gemm_grouped(problems) -> List[torch.Tensor]:
    """Several independent GEMMs in one persistent launch (``lb_gemm_grouped``): short tiles of one
    problem fill the idle tail of another.  ``problems``: up to 8 tuples
    ``(a, b, a_mn, b_mn, out_or_None, accumulate)`` with the conventions of :func:`gemm`;
    ``accumulate`` adds the product to the old contents of ``out``.  A tuple may carry three more
    entries ``(epi, c2, half)`` that select a SwiGLU epilogue: ``epi = 1`` (``b`` is a fused
    ``[2 * half, K]`` gate | up weight; ``out [M, 2 * half]`` receives g | u and ``c2 [M, half]``
    receives ``silu(g) * u``) or ``epi = 2`` (the product is the gradient of ``silu(g) * u``; ``c2``
    holds g | u and ``out [M, 2 * half]`` receives dg | du).  Returns the outputs."""
    n = len(problems)
    assert 1 <= n <= 8
    import ctypes
    PA, IA, LA = ctypes.c_void_p * n, ctypes.c_int * n, ctypes.c_longlong * n
    A, B, C, C2 = PA(), PA(), PA(), PA()
    M, N, K, amn, bmn, acc, epi, half = IA(), IA(), IA(), IA(), IA(), IA(), IA(), IA()
    lda, ldb, ldc, ldc2 = LA(), LA(), LA(), LA()
    outs = []
    any_epi = False
    for i, prob in enumerate(problems):
        a, b, a_mn, b_mn, out, accumulate = prob[:6]
        e, c2, hf = prob[6:9] if len(prob) > 6 else (0, None, 0)
        assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
        m, k = (a.shape[1], a.shape[0]) if a_mn else a.shape
        nn_, kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
        assert k == kb, f"K mismatch {k} vs {kb}"
        if out is None:
            assert not accumulate
            out = torch.empty(m, 2 * hf if e == 2 else nn_, dtype=a.dtype, device=a.device)
        A[i], B[i], C[i] = a.data_ptr(), b.data_ptr(), out.data_ptr()
        M[i], N[i], K[i] = m, nn_, k
        lda[i], ldb[i], ldc[i] = a.stride(0), b.stride(0), out.stride(0)
        amn[i], bmn[i], acc[i] = int(a_mn), int(b_mn), int(accumulate)
        epi[i], half[i] = int(e), int(hf)
        if e:
            any_epi = True
            assert c2 is not None and c2.stride(1) == 1 and c2.shape[0] == m and out.shape[1] == 2 * hf
            assert c2.shape[1] == (hf if e == 1 else 2 * hf)
            C2[i], ldc2[i] = c2.data_ptr(), c2.stride(0)
        outs.append(out)
    if any_epi:
        native.call("lb_gemm_grouped_epi", n, A, B, C, M, N, K, lda, ldb, ldc, amn, bmn, acc, epi, C2, ldc2, half,
                    native.stream_ptr())
    else:
        native.call("lb_gemm_grouped", n, A, B, C, M, N, K, lda, ldb, ldc, amn, bmn, acc, native.stream_ptr())
    return outs


# ---- deferred weight gradients ------------------------------------------------------------------
# A lone weight-gradient GEMM often fills the 148 SMs badly (a [1280, 2048] gradient is 80 tiles).
# Ops whose parameters' gradients live in the optimizer's arena may queue the product instead of
# launching it; the queue is flushed as ONE grouped launch (tiles of several gradients share the
# waves) at the latest when the backward pass ends, and the optimizer's bucket callbacks run then.

_WQ: List[tuple] = []
_WQ_STATE = {"callback": False}
_DEFER_WGRAD = os.environ.get("LIGHTRON_DEFER_WGRAD", "1") != "0"


def direct_wgrad_ok(params) -> bool:
    """True when every weight's ``.grad`` is a row-adjacent view of the bf16 gradient arena."""
    return bool(params) and all(getattr(w, "_lb_direct_grad", False) and w.grad is not None for w in params) \
        and _rows_adjacent([w.grad for w in params])


def wgrad_queue_uses(tag) -> bool:
    return any(t == tag for *_rest, t in _WQ)


def defer_wgrad(dy2: torch.Tensor, x2: torch.Tensor, params, tag=None) -> None:
    """Queue  grad(params) += dy2^T x2  (dy2 [tokens, sum n_i], x2 [tokens, K]).  ``tag`` lets the
    caller ask later whether an entry with that tag is still pending (buffers that get recycled)."""
    for w in params:
        w._lb_wgrad_pending = True
    _WQ.append((dy2, x2, tuple(params), tag))
    if not _WQ_STATE["callback"]:
        _WQ_STATE["callback"] = True
        torch.autograd.Variable._execution_engine.queue_callback(flush_wgrads)
    if len(_WQ) >= 8:
        flush_wgrads(final=False)


def flush_wgrads(final: bool = True) -> None:
    if final:
        _WQ_STATE["callback"] = False
    if not _WQ:
        return
    items = list(_WQ)
    _WQ.clear()
    gemm_grouped([(dy2, x2, True, True, _as_strided_cat([w.grad for w in params]), True)
                  for dy2, x2, params, _tag in items])
    for _dy2, _x2, params, _tag in items:
        for w in params:
            w._lb_wgrad_pending = False
            for hook in getattr(w, "_lb_grad_hooks", ()):
                hook(w)


_GROUP_BWD = os.environ.get("LIGHTRON_GROUPED_BWD", "1") != "0"
_DIRECT_WGRAD = os.environ.get("LIGHTRON_DIRECT_WGRAD", "1") != "0"


class _Linear(torch.autograd.Function):
    """y = x W^T for one weight or several row-adjacent weights (fused QKV / gate+up)."""

    @staticmethod
    def forward(ctx, x, *ws):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.fused = _rows_adjacent(ws)
        ctx.save_for_backward(x2, *ws)
        ctx.params = ws
        ctx.xshape = x.shape
        if ctx.fused:
            y = gemm(x2, _as_strided_cat(ws))
        else:
            y = torch.cat([gemm(x2, w) for w in ws], dim=1)
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x2, *ws = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx, dws = _linear_backward(x2, ws, ctx.params, dy2, ctx.fused, ctx.needs_input_grad[0], ctx.needs_input_grad[1:])
        return (None if dx is None else dx.view(ctx.xshape), *dws)


def _linear_backward(x2, ws, params, dy2, fused, need_x, need_ws):
    """Gradients of ``y = x2 [W_0; W_1; ...]^T``: (dx2 or None, one entry per weight; None where the
    gradient was accumulated straight into the optimizer's arena)."""
    sizes = [w.shape[0] for w in ws]
    dx = None
    if _GROUP_BWD and fused and need_x and any(need_ws):
        # data gradient and weight gradient in one launch: the short dgrad tiles fill the
        # last, partly empty wave of the wgrad
        if _DIRECT_WGRAD and all(need_ws) and direct_wgrad_ok(params):
            # the weight gradient accumulates straight into the gradient arena in the GEMM
            # epilogue: no separate add, and the optimizer's bucket hooks are called by hand
            gout = _as_strided_cat([w.grad for w in params])
            dx = gemm_grouped([(dy2, x2, True, True, gout, True),
                               (dy2, _as_strided_cat(ws), False, True, None, False)])[1]
            for w in params:
                for hook in getattr(w, "_lb_grad_hooks", ()):
                    hook(w)
            return dx, [None] * len(ws)
        dx, dw = gemm_grouped([(dy2, x2, True, True, None, False),
                               (dy2, _as_strided_cat(ws), False, True, None, False)])[::-1]
        dws, off = [], 0
        for n in sizes:
            dws.append(dw[off:off + n])
            off += n
        return dx, dws
    if need_x:
        if fused:
            dx = gemm(dy2, _as_strided_cat(ws), b_mn=True)
        else:
            off = 0
            for w, n in zip(ws, sizes):
                part = gemm(dy2[:, off:off + n], w, b_mn=True)
                dx = part if dx is None else dx.add_(part)
                off += n
    dws: List[Optional[torch.Tensor]] = [None] * len(ws)
    if any(need_ws):
        dw = gemm(dy2, x2, a_mn=True, b_mn=True)        # [sum n_i, K]
        off = 0
        for i, n in enumerate(sizes):
            dws[i] = dw[off:off + n]
            off += n
    return dx, dws


_FUSED_SWIGLU = os.environ.get("LIGHTRON_FUSED_SWIGLU", "1") != "0"


class _SwiGLUMLP(torch.autograd.Function):
    """``(silu(x W1^T) * (x W3^T)) W2^T`` with the activation inside the GEMM epilogues: the gate | up
    GEMM writes ``silu(g) * u`` next to g | u, and the data-gradient GEMM of the down projection
    turns its tile of dh into dg | du before storing, so neither the activation nor its gradient is
    a pass of its own (model/model.py:69 of the reference is ``w2(F.silu(w1(x)) * w3(x))``)."""

    @staticmethod
    def forward(ctx, x, w1, w3, w2):
        x2 = x.reshape(-1, x.shape[-1])
        F_ = w1.shape[0]
        gu = torch.empty(x2.shape[0], 2 * F_, dtype=x.dtype, device=x.device)
        h = torch.empty(x2.shape[0], F_, dtype=x.dtype, device=x.device)
        gemm_grouped([(x2, _as_strided_cat((w1, w3)), False, False, gu, False, 1, h, F_)])
        y = gemm(h, w2)
        ctx.save_for_backward(x2, gu, h, w1, w3, w2)
        ctx.params = (w1, w3, w2)
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x2, gu, h, w1, w3, w2 = ctx.saved_tensors
        p1, p3, p2 = ctx.params
        F_ = w1.shape[0]
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        need = ctx.needs_input_grad
        dgu = torch.empty_like(gu)
        act = (dy2, w2, False, True, dgu, False, 2, gu, F_)          # dh = dy W2, stored as dg | du
        dw2 = None
        if need[3] and _DIRECT_WGRAD and direct_wgrad_ok((p2,)):
            gemm_grouped([(dy2, h, True, True, p2.grad, True), act])
            for hook in getattr(p2, "_lb_grad_hooks", ()):
                hook(p2)
        elif need[3]:
            dw2 = gemm_grouped([(dy2, h, True, True, None, False), act])[0]
        else:
            gemm_grouped([act])
        dx, (dw1, dw3) = _linear_backward(x2, (w1, w3), (p1, p3), dgu, True, need[0], need[1:3])
        return (None if dx is None else dx.view(ctx.xshape), dw1, dw3, dw2)


def swiglu_mlp_ok(x: torch.Tensor, w1, w3, w2) -> bool:
    return bool(_FUSED_SWIGLU and native.use_native(x) and x.shape[-1] % 8 == 0 and w1.shape[0] % 8 == 0
                and w2.shape[0] % 8 == 0 and w1.shape == w3.shape and _rows_adjacent((w1, w3)) and w2.is_contiguous())


def swiglu_mlp(x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """``w2(silu(w1 x) * w3 x)`` for [n, K] weights; the fused-epilogue kernels when they apply."""
    if swiglu_mlp_ok(x, w1, w3, w2):
        return _SwiGLUMLP.apply(x, w1, w3, w2)
    return linear(swiglu(linear(x, w1, w3)), w2)


def _grouped_launch(problems) -> None:
    for i in range(0, len(problems), 8):
        gemm_grouped(problems[i:i + 8])


class _GroupedLinear(torch.autograd.Function):
    """Row segments of ``x`` times different weights: segment e (``counts[e]`` rows) uses the
    row-adjacent weights ``groups[e]``.  All segments run in one grouped launch (forward: one
    problem per segment; backward: data and weight gradient of every segment together)."""

    @staticmethod
    def forward(ctx, x, counts, per_group, *flat_ws):
        groups = [flat_ws[i:i + per_group] for i in range(0, len(flat_ws), per_group)]
        N = sum(w.shape[0] for w in groups[0])
        y = torch.empty(x.shape[0], N, dtype=x.dtype, device=x.device)
        probs, off = [], 0
        for c, ws in zip(counts, groups):
            if c:
                probs.append((x[off:off + c], _as_strided_cat(ws), False, False, y[off:off + c], False))
            off += c
        if off < x.shape[0]:
            y[off:].zero_()
        _grouped_launch(probs)
        ctx.save_for_backward(x, *flat_ws)
        ctx.counts, ctx.per_group, ctx.params = list(counts), per_group, flat_ws
        return y

    @staticmethod
    def backward(ctx, dy):
        x, *flat_ws = ctx.saved_tensors
        per = ctx.per_group
        groups = [flat_ws[i:i + per] for i in range(0, len(flat_ws), per)]
        pgroups = [ctx.params[i:i + per] for i in range(0, len(flat_ws), per)]
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        direct = _DIRECT_WGRAD and all(ctx.needs_input_grad[3:]) and all(direct_wgrad_ok(pg) for pg in pgroups)
        probs, dws, off = [], [], 0
        for c, ws, pg in zip(ctx.counts, groups, pgroups):
            if direct:
                gout, acc = (_as_strided_cat([w.grad for w in pg]), True)
            else:
                gout, acc = (torch.zeros(sum(w.shape[0] for w in ws), x.shape[1], dtype=x.dtype, device=x.device), False)
                dws.append(gout)
            if c:
                probs.append((dy[off:off + c], x[off:off + c], True, True, gout, acc))           # wgrad first: longest tiles
                probs.append((dy[off:off + c], _as_strided_cat(ws), False, True, dx[off:off + c], False))
            off += c
        if off < x.shape[0]:
            dx[off:].zero_()
        _grouped_launch(probs)
        if direct:
            for pg in pgroups:
                for w in pg:
                    for hook in getattr(w, "_lb_grad_hooks", ()):
                        hook(w)
            return (dx, None, None, *([None] * len(flat_ws)))
        out = []
        for dw, ws in zip(dws, groups):
            o = 0
            for w in ws:
                out.append(dw[o:o + w.shape[0]])
                o += w.shape[0]
        return (dx, None, None, *out)


def grouped_linear_ok(x: torch.Tensor, groups) -> bool:
    return bool(native.use_native(x) and x.shape[-1] % 8 == 0 and groups
                and all(_rows_adjacent(ws) and all(w.shape[0] % 8 == 0 for w in ws) for ws in groups))


def grouped_linear(x: torch.Tensor, counts, groups) -> torch.Tensor:
    """x [R, K], rows sorted by segment; segment e has ``counts[e]`` rows and is multiplied by the
    weights ``groups[e]`` (a tuple of [n_i, K] matrices whose outputs are concatenated, as in
    :func:`linear`).  Rows beyond ``sum(counts)`` give zeros.  The per-expert GEMM of a MoE layer
    (one launch for all local experts; the reference applies a single expert, model/model.py:109)."""
    if grouped_linear_ok(x, groups):
        flat = [w for ws in groups for w in ws]
        return _GroupedLinear.apply(x, list(counts), len(groups[0]), *flat)
    outs, off = [], 0
    for c, ws in zip(counts, groups):
        outs.append(linear(x[off:off + c], *ws))
        off += c
    if off < x.shape[0]:
        outs.append(x.new_zeros(x.shape[0] - off, outs[0].shape[1]))
    return torch.cat(outs, dim=0)


def linear(x: torch.Tensor, *ws: torch.Tensor) -> torch.Tensor:
    """x [..., K] times one or more [n_i, K] weights -> [..., sum n_i]."""
    if native.use_native(x) and x.shape[-1] % 8 == 0 and all(w.shape[0] % 8 == 0 for w in ws):
        return _Linear.apply(x, *ws)
    # CPU / fp32 oracle path, and GEMMs whose widths are not multiples of 8 (a MoE router with
    # fewer than 8 experts): TMA needs 16-byte rows, and such a GEMM is tiny anyway
    if len(ws) == 1:
        return F.linear(x, ws[0])
    return torch.cat([F.linear(x, w) for w in ws], dim=-1)


# --------------------------------------------------------------------------------------
# RMSNorm (optionally fused with the residual add that precedes it)
# --------------------------------------------------------------------------------------


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, w, eps):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows, cols = x2.shape
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        if res is not None:
            r2 = res.reshape(-1, shape[-1])
            if not r2.is_contiguous():
                r2 = r2.contiguous()
            h = torch.empty_like(x2)
        else:
            r2, h = None, None
        native.call("lb_rmsnorm_fwd", x2.data_ptr(), native.ptr(r2), w.data_ptr(), native.ptr(h), y.data_ptr(),
                    rstd.data_ptr(), rows, cols, float(eps), native.stream_ptr())
        src = h if res is not None else x2
        ctx.save_for_backward(src, w, rstd)
        ctx.has_res = res is not None
        ctx.shape = shape
        if res is not None:
            return h.view(shape), y.view(shape)
        return y.view(shape)

    @staticmethod
    def backward(ctx, *grads):
        src, w, rstd = ctx.saved_tensors
        rows, cols = src.shape
        if ctx.has_res:
            dh, dy = grads
        else:
            dh, dy = None, grads[0]
        dy2 = dy.reshape(rows, cols)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dh2 = None
        if dh is not None:
            dh2 = dh.reshape(rows, cols)
            if not dh2.is_contiguous():
                dh2 = dh2.contiguous()
        lib = native.require()
        nblk = lib.lb_rmsnorm_bwd_blocks(rows, cols)
        partial = torch.empty(nblk, cols, dtype=torch.float32, device=src.device)
        dx = torch.empty_like(src)
        dw = torch.empty_like(w)
        native.call("lb_rmsnorm_bwd", dy2.data_ptr(), src.data_ptr(), w.data_ptr(), rstd.data_ptr(), native.ptr(dh2),
                    dx.data_ptr(), partial.data_ptr(), dw.data_ptr(), rows, cols, nblk, native.stream_ptr())
        dxv = dx.view(ctx.shape)
        if ctx.has_res:
            return dxv, dxv, dw, None
        return dxv, None, dw, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    if native.use_native(x):
        return _RMSNorm.apply(x, None, w, eps)
    return ref.rmsnorm(x, w, eps)


def add_rmsnorm(x: torch.Tensor, res: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """h = x + res; y = rmsnorm(h).  Returns (h, y) from one pass over memory."""
    if native.use_native(x):
        return _RMSNorm.apply(x, res, w, eps)
    h = x + res
    return h, ref.rmsnorm(h, w, eps)


# --------------------------------------------------------------------------------------
# RoPE
# --------------------------------------------------------------------------------------


def _rope_native_(t: torch.Tensor, cos, sin, positions, S: int, n_heads: int, head_dim: int, inverse: bool) -> None:
    """In place on a [T, *] row-major view whose first n_heads*head_dim columns are heads."""
    T = t.shape[0]
    native.call("lb_rope", t.data_ptr(), cos.data_ptr(), sin.data_ptr(), native.ptr(positions), T, S, n_heads,
                head_dim, t.stride(0), int(inverse), native.stream_ptr())


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, positions):
        B, S, h, d = x.shape
        out = x.contiguous().clone()
        _rope_native_(out.view(B * S, h * d), cos, sin, positions, S, h, d, False)
        ctx.save_for_backward(cos, sin, positions)
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin, positions = ctx.saved_tensors
        B, S, h, d = dy.shape
        dx = dy.contiguous().clone()
        _rope_native_(dx.view(B * S, h * d), cos, sin, positions, S, h, d, True)
        return dx, None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: Optional[torch.Tensor] = None):
    """x [B, S, h, d] -> rotated copy.  ``positions`` [S] int32 picks table rows."""
    if native.use_native(x):
        if positions is not None and positions.dtype != torch.int32:
            positions = positions.to(torch.int32)
        return _Rope.apply(x, cos, sin, positions)
    return ref.rope(x, cos, sin, positions)


# --------------------------------------------------------------------------------------
# SwiGLU on a fused [T, 2I] gate|up tensor
# --------------------------------------------------------------------------------------


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        shape = gu.shape
        gu2 = gu.reshape(-1, shape[-1])
        I = shape[-1] // 2
        out = torch.empty(gu2.shape[0], I, dtype=gu.dtype, device=gu.device)
        native.call("lb_swiglu_fwd", gu2.data_ptr(), out.data_ptr(), gu2.shape[0], I, gu2.stride(0), native.stream_ptr())
        ctx.save_for_backward(gu2)
        ctx.shape = shape
        return out.view(*shape[:-1], I)

    @staticmethod
    def backward(ctx, dy):
        (gu2,) = ctx.saved_tensors
        I = gu2.shape[1] // 2
        dy2 = dy.reshape(-1, I)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dgu = torch.empty(gu2.shape[0], 2 * I, dtype=gu2.dtype, device=gu2.device)
        native.call("lb_swiglu_bwd", gu2.data_ptr(), dy2.data_ptr(), dgu.data_ptr(), gu2.shape[0], I, gu2.stride(0),
                    native.stream_ptr())
        return dgu.view(ctx.shape)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """gu [..., 2I] holding gate | up -> silu(gate) * up [..., I]."""
    if native.use_native(gu):
        return _SwiGLU.apply(gu)
    I = gu.shape[-1] // 2
    return ref.swiglu(gu[..., :I], gu[..., I:])


# --------------------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------------------


def _layout_ok(t: torch.Tensor) -> bool:
    B, S, h, d = t.shape
    return t.stride(3) == 1 and t.stride(2) == d and (B == 1 or t.stride(0) == S * t.stride(1)) \
        and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0


def _check_attn_layout(t: torch.Tensor) -> None:
    if not _layout_ok(t):
        raise ValueError(f"attention operand must be [B,S,h,d] with unit inner stride, head stride d, batch "
                         f"stride S*token_stride and 16-byte aligned rows; got shape {tuple(t.shape)} "
                         f"strides {t.stride()}")


def _fix_layout(t: torch.Tensor) -> torch.Tensor:
    return t if _layout_ok(t) else t.contiguous()


def flash_fwd_native(q, k, v, causal: bool, scale: float):
    q, k, v = _fix_layout(q), _fix_layout(k), _fix_layout(v)
    B, Sq, hq, d = q.shape
    Sk, hkv = k.shape[1], k.shape[2]
    o = torch.empty(B, Sq, hq, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, hq, Sq, dtype=torch.float32, device=q.device)
    # head_dim 64 / 128 run on the tcgen05 kernel; 32 (and causal with Sk < Sq) on the mma.sync one
    use_tc = d in (64, 128) and not (causal and Sk < Sq) and os.environ.get("LIGHTRON_FA", "tc") == "tc"
    native.call("lb_flash_fwd_tc" if use_tc else "lb_flash_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                B, Sq, Sk, hq, hkv, d, q.stride(1), k.stride(1), v.stride(1), o.stride(1), float(scale), int(causal),
                native.stream_ptr())
    return o, lse


def flash_bwd_native(q, k, v, o, lse, do, causal: bool, scale: float, dq=None, dk=None, dv=None):
    """Returns (dq, dk, dv).  Output tensors may be caller-provided strided views."""
    B, Sq, hq, d = q.shape
    Sk, hkv = k.shape[1], k.shape[2]
    if dq is None:
        dq = torch.empty(B, Sq, hq, d, dtype=q.dtype, device=q.device)
    if dk is None:
        dk = torch.empty(B, Sk, hkv, d, dtype=q.dtype, device=q.device)
    if dv is None:
        dv = torch.empty(B, Sk, hkv, d, dtype=q.dtype, device=q.device)
    q, k, v, o, do = (_fix_layout(t) for t in (q, k, v, o, do))
    lse = lse.contiguous()
    for t in (dq, dk, dv):
        _check_attn_layout(t)
    delta = torch.empty(B, hq, Sq, dtype=torch.float32, device=q.device)
    use_tc = d in (64, 128) and not (causal and Sk < Sq) and os.environ.get("LIGHTRON_FA_BWD", "tc") == "tc"
    # fp32 dQ accumulator: the tcgen05 kernel uses a tile-permuted layout padded to 128-row tiles
    n_acc = B * hq * ((Sq + 127) // 128) * 128 * d if use_tc else B * Sq * hq * d
    dq_acc = torch.zeros(n_acc, dtype=torch.float32, device=q.device)
    native.call("lb_flash_bwd_tc" if use_tc else "lb_flash_bwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                B, Sq, Sk, hq, hkv, d, q.stride(1), k.stride(1), v.stride(1), o.stride(1), do.stride(1),
                dq.stride(1), dk.stride(1), dv.stride(1), float(scale), int(causal), native.stream_ptr())
    return dq, dk, dv


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        o, lse = flash_fwd_native(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale = causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = flash_bwd_native(q, k, v, o, lse, do, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


def flash_attention(q, k, v, causal: bool = True, scale: Optional[float] = None):
    """q [B,Sq,hq,d], k/v [B,Sk,hkv,d] -> [B,Sq,hq,d]; GQA by indexing (no repeat_kv)."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if native.use_native(q):
        return _FlashAttn.apply(q, k, v, causal, scale)
    return ref.attention(q, k, v, causal=causal, scale=scale)


class _RopeAttnQKV(torch.autograd.Function):
    """RoPE + causal attention straight on the fused projection output [B*S, (hq+2hkv)*d].
    Forward rotates q and k in place inside ``qkv`` without telling autograd: the producer is
    a GEMM whose backward needs its inputs, not this output, and nothing else may consume the
    tensor (the caller hands over ownership).  Backward writes one dqkv tensor and un-rotates
    its q,k columns in place, so no slice/concat copies exist on either side."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, B, S, hq, hkv, d, scale):
        T = B * S
        qkv2 = qkv.view(T, (hq + 2 * hkv) * d)
        _rope_native_(qkv2, cos, sin, positions, S, hq + hkv, d, False)
        row = qkv2.stride(0)
        off = qkv2.storage_offset()
        q = qkv2.as_strided((B, S, hq, d), (S * row, row, d, 1), off)
        k = qkv2.as_strided((B, S, hkv, d), (S * row, row, d, 1), off + hq * d)
        v = qkv2.as_strided((B, S, hkv, d), (S * row, row, d, 1), off + (hq + hkv) * d)
        o, lse = flash_fwd_native(q, k, v, True, scale)
        ctx.save_for_backward(qkv, o, lse, cos, sin, positions)
        ctx.dims = (B, S, hq, hkv, d, scale)
        return o.view(T, hq * d)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, cos, sin, positions = ctx.saved_tensors
        B, S, hq, hkv, d, scale = ctx.dims
        T = B * S
        qkv2 = qkv.view(T, (hq + 2 * hkv) * d)
        row = qkv2.stride(0)
        off = qkv2.storage_offset()
        q = qkv2.as_strided((B, S, hq, d), (S * row, row, d, 1), off)
        k = qkv2.as_strided((B, S, hkv, d), (S * row, row, d, 1), off + hq * d)
        v = qkv2.as_strided((B, S, hkv, d), (S * row, row, d, 1), off + (hq + hkv) * d)
        dqkv = torch.empty(T, (hq + 2 * hkv) * d, dtype=qkv2.dtype, device=qkv2.device)
        drow = dqkv.stride(0)
        dq = dqkv.as_strided((B, S, hq, d), (S * drow, drow, d, 1), 0)
        dk = dqkv.as_strided((B, S, hkv, d), (S * drow, drow, d, 1), hq * d)
        dv = dqkv.as_strided((B, S, hkv, d), (S * drow, drow, d, 1), (hq + hkv) * d)
        flash_bwd_native(q, k, v, o, lse, do.reshape(B, S, hq, d), True, scale, dq, dk, dv)
        _rope_native_(dqkv, cos, sin, positions, S, hq + hkv, d, True)
        return dqkv.view(qkv.shape), None, None, None, None, None, None, None, None, None


def rope_attention_qkv(qkv: torch.Tensor, cos, sin, positions, B: int, S: int, hq: int, hkv: int, d: int,
                       scale: Optional[float] = None) -> torch.Tensor:
    """qkv [B*S, (hq+2hkv)*d] (q heads | k heads | v heads per token) -> attention output
    [B*S, hq*d] with RoPE applied to q and k.  Causal, full sequence local."""
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if native.use_native(qkv):
        if positions is not None and positions.dtype != torch.int32:
            positions = positions.to(torch.int32)
        return _RopeAttnQKV.apply(qkv, cos, sin, positions, B, S, hq, hkv, d, scale)
    T = B * S
    q, k, v = qkv.view(T, -1).split([hq * d, hkv * d, hkv * d], dim=-1)
    q = ref.rope(q.reshape(B, S, hq, d), cos, sin, positions)
    k = ref.rope(k.reshape(B, S, hkv, d), cos, sin, positions)
    o = ref.attention(q, k, v.reshape(B, S, hkv, d), causal=True, scale=scale)
    return o.reshape(T, hq * d)


# --------------------------------------------------------------------------------------
# Embedding (optionally vocab-parallel)
# --------------------------------------------------------------------------------------


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, w, vocab_start):
        T = tokens.numel()
        H = w.shape[1]
        out = torch.empty(T, H, dtype=w.dtype, device=w.device)
        tok = tokens.reshape(-1).contiguous()
        native.call("lb_embedding_fwd", tok.data_ptr(), w.data_ptr(), out.data_ptr(), T, H, vocab_start,
                    vocab_start + w.shape[0], native.stream_ptr())
        ctx.save_for_backward(tok)
        ctx.wshape, ctx.vocab_start = w.shape, vocab_start
        return out.view(*tokens.shape, H)

    @staticmethod
    def backward(ctx, dy):
        (tok,) = ctx.saved_tensors
        V, H = ctx.wshape
        dy2 = dy.reshape(-1, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dw = torch.zeros(V, H, dtype=dy.dtype, device=dy.device)
        native.call("lb_embedding_bwd", tok.data_ptr(), dy2.data_ptr(), dw.data_ptr(), tok.numel(), H,
                    ctx.vocab_start, ctx.vocab_start + V, native.stream_ptr())
        return None, dw, None


def embedding(tokens: torch.Tensor, w: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Rows of ``w`` (which holds vocab ids [vocab_start, vocab_start + w.shape[0])); ids outside
    the range give zero rows (vocab-parallel partial result, parallel/parallel_tp.py:131-143)."""
    if native.use_native(w):
        return _Embedding.apply(tokens, w, vocab_start)
    local = tokens - vocab_start
    mask = (local < 0) | (local >= w.shape[0])
    out = F.embedding(local.masked_fill(mask, 0), w)
    if vocab_start != 0 or bool(mask.any()):
        out = out.masked_fill(mask.unsqueeze(-1), 0.0)
    return out


# --------------------------------------------------------------------------------------
# Cross-entropy, vocab-parallel aware: ranks exchange (max, sum-exp, target logit) per token,
# never logits (the reference all-gathers [B,S,V] logits: parallel/parallel_tp.py:31,72).
# --------------------------------------------------------------------------------------


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, vocab_start, group, n_valid_total, ignore_index):
        T, V = logits.shape
        use_native = native.use_native(logits)
        tgt = targets.reshape(-1).contiguous()
        if use_native:
            mx = torch.empty(T, dtype=torch.float32, device=logits.device)
            se = torch.empty(T, dtype=torch.float32, device=logits.device)
            tl = torch.empty(T, dtype=torch.float32, device=logits.device)
            native.call("lb_ce_stats", logits.data_ptr(), tgt.data_ptr(), mx.data_ptr(), se.data_ptr(), tl.data_ptr(),
                        T, V, logits.stride(0), vocab_start, native.stream_ptr())
        else:
            lf = logits.float()
            mx = lf.max(dim=-1).values
            se = torch.exp(lf - mx[:, None]).sum(-1)
            local = tgt - vocab_start
            inr = (local >= 0) & (local < V)
            tl = torch.where(inr, lf.gather(1, local.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(mx))
        if group is not None and dist.get_world_size(group) > 1:
            gmx = mx.clone()
            dist.all_reduce(gmx, op=dist.ReduceOp.MAX, group=group)
            packed = torch.stack((se * torch.exp(mx - gmx), tl))
            dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
            se, tl, mx = packed[0], packed[1], gmx
        lse = mx + torch.log(se)
        valid = tgt != ignore_index
        n_valid = n_valid_total if n_valid_total is not None else int(valid.sum().item())
        per_tok = torch.where(valid, lse - tl, torch.zeros_like(lse))
        loss = per_tok.sum() / max(n_valid, 1)
        ctx.save_for_backward(logits, tgt, lse)
        ctx.meta = (vocab_start, n_valid, ignore_index, use_native)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits, tgt, lse = ctx.saved_tensors
        vocab_start, n_valid, ignore_index, use_native = ctx.meta
        T, V = logits.shape
        if use_native:
            # dlogits overwrites the logits buffer: it is dead after the loss, and at
            # [16384, 32000] it is the largest activation of the step.
            dl = dloss.float().reshape(1).contiguous()      # read on the device: no host sync
            native.call("lb_ce_grad", logits.data_ptr(), tgt.data_ptr(), lse.data_ptr(), logits.data_ptr(),
                        dl.data_ptr(), T, V, logits.stride(0), vocab_start, 1.0 / max(n_valid, 1), ignore_index,
                        native.stream_ptr())
            return logits, None, None, None, None, None
        p = torch.exp(logits.float() - lse[:, None])
        local = tgt - vocab_start
        inr = (local >= 0) & (local < V)
        idx = torch.nonzero(inr, as_tuple=False)[:, 0]
        p[idx, local[idx]] -= 1.0
        p = p * (tgt != ignore_index)[:, None]
        return (p * (dloss.float() / max(n_valid, 1))).to(logits.dtype), None, None, None, None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int = 0, group=None,
                  n_valid_total: Optional[int] = None, ignore_index: int = -100) -> torch.Tensor:
    """Mean NLL of [T, V_local] logits.  With ``group`` the vocab dim is sharded across it.
    ``n_valid_total`` (the number of non-ignored targets) avoids a host sync when known."""
    logits2 = logits.reshape(-1, logits.shape[-1])
    return _CrossEntropy.apply(logits2, targets, vocab_start, group, n_valid_total, ignore_index)
