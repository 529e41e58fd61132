"""Plain PyTorch restatement of every hot op.  It is (a) the numeric oracle that the CUDA
kernels are tested against, (b) the CPU / gloo execution path and (c) the "library" baseline.

Math follows the reference model: RMSNorm computed in fp32 then cast then scaled
(``layers/layers.py:11-16``), RoPE on interleaved pairs (``layers/layers.py:18-24,44-70``),
SwiGLU ``silu(w1 x) * w3 x`` (``model/model.py:69``), causal softmax attention with scale
1/sqrt(d) (``model/model.py:193-198``) and token-mean cross-entropy (``trainer.py:52``).
GQA is handled by indexing, not by materialising repeated KV (``model/model.py:11-34``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y.type_as(x) * weight


def rope_tables(head_dim: int, end: int, theta: float = 10000.0,
                device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [end, head_dim/2] in fp32 (kept real so a dtype cast of the model cannot
    drop the imaginary part, which happens to the reference's complex buffer under bf16)."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device)[: head_dim // 2].float() / head_dim))
    t = torch.arange(end, device=device).float()
    ang = torch.outer(t, freqs)
    return torch.cos(ang), torch.sin(ang)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
         positions: Optional[torch.Tensor] = None, inverse: bool = False) -> torch.Tensor:
    """x: [B, S, h, d]; rotates pairs (x[2i], x[2i+1]) by angle pos * theta^(-2i/d).
    ``positions`` [S] selects table rows (context parallel shards); default arange(S).
    ``inverse`` applies the transpose rotation (the backward of RoPE)."""
    B, S, h, d = x.shape
    if positions is None:
        c, s = cos[:S], sin[:S]
    else:
        c, s = cos[positions], sin[positions]
    c = c.view(1, S, 1, d // 2).float()
    s = s.view(1, S, 1, d // 2).float()
    if inverse:
        s = -s
    xf = x.float().reshape(B, S, h, d // 2, 2)
    x0, x1 = xf[..., 0], xf[..., 1]
    out = torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), dim=-1)
    return out.reshape(B, S, h, d).type_as(x)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return (F.silu(gate.float()) * up.float()).type_as(gate)


def swiglu_bwd(gate, up, dy):
    g, u, d = gate.float(), up.float(), dy.float()
    sig = torch.sigmoid(g)
    dgate = d * u * sig * (1 + g * (1 - sig))
    dup = d * g * sig
    return dgate.type_as(gate), dup.type_as(up)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              scale: Optional[float] = None, q_pos: Optional[torch.Tensor] = None,
              k_pos: Optional[torch.Tensor] = None, return_lse: bool = False):
    """q: [B, Sq, hq, d]; k, v: [B, Sk, hkv, d] -> [B, Sq, hq, d].  fp32 math.
    With ``q_pos``/``k_pos`` (global positions) the causal mask is q_pos >= k_pos, which is what
    context-parallel shards need."""
    B, Sq, hq, d = q.shape
    Sk, hkv = k.shape[1], k.shape[2]
    rep = hq // hkv
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3).reshape(B, hkv, rep, Sq, d)
    kf = k.float().permute(0, 2, 1, 3)                      # [B, hkv, Sk, d]
    vf = v.float().permute(0, 2, 1, 3)
    s = torch.einsum("bgrqd,bgkd->bgrqk", qf, kf) * scale
    if causal:
        qp = torch.arange(Sq, device=q.device) + (Sk - Sq) if q_pos is None else q_pos
        kp = torch.arange(Sk, device=q.device) if k_pos is None else k_pos
        mask = qp[:, None] >= kp[None, :]
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                         # [B, hkv, rep, Sq]
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)                        # fully masked rows
    o = torch.einsum("bgrqk,bgkd->bgrqd", p, vf)
    o = o.reshape(B, hq, Sq, d).permute(0, 2, 1, 3).type_as(q)
    if return_lse:
        return o, lse.reshape(B, hq, Sq)
    return o


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Token-mean NLL over [T, V] logits (fp32 math)."""
    return F.cross_entropy(logits.float(), targets, reduction="mean", ignore_index=ignore_index)


def adamw_step(p, g, m, v, lr, beta1, beta2, eps, wd, step):
    """One decoupled-weight-decay Adam update in fp32 (torch.optim.AdamW semantics)."""
    g = g.float()
    p.mul_(1 - lr * wd)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
