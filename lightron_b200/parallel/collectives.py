"""Stand-alone ring collectives built from point-to-point messages.

Parity with the reference's hand-rolled primitives: ``ring_all_reduce``
(parallel/communication/all_reduce.py:26-93: flatten + pad, N-1 reduce-scatter steps, N-1
all-gather steps), ``ring_all_gather`` (ring_all_gather.py:25-57), ``ring_reduce_scatter``
(ring_reduce_scatter.py:25-67: list of chunks in, rank r ends with the sum of chunk r) and
``ring_p2p`` (ring_p2p.py:25-38).  They run on any backend (NCCL on GPUs, gloo on CPU ranks),
inside any process group, and are checked against the library collectives in the tests, which
is what the reference's test scripts do by printing a difference.

On a single NVSwitch box every GPU reaches every peer at full bandwidth, so rings are not the
fast path of this framework (the fused peer-memory kernels are); these functions exist for API
parity, as an oracle that does not depend on the library collectives, and for backends that lack
a collective.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _ring(group):
    n = dist.get_world_size(group)
    r = dist.get_rank(group)
    nxt = dist.get_global_rank(group, (r + 1) % n) if group is not None else (r + 1) % n
    prv = dist.get_global_rank(group, (r - 1) % n) if group is not None else (r - 1) % n
    return n, r, nxt, prv


def _sendrecv(send: torch.Tensor, recv: torch.Tensor, nxt: int, prv: int, group, rank: int) -> None:
    ops = [dist.P2POp(dist.isend, send, nxt, group), dist.P2POp(dist.irecv, recv, prv, group)]
    if rank % 2:
        ops.reverse()
    for req in dist.batch_isend_irecv(ops):
        req.wait()


def ring_p2p(tensor: torch.Tensor, src: int, dst: int, group=None) -> torch.Tensor:
    """Send ``tensor`` from group rank ``src`` to group rank ``dst`` (in place on ``dst``)."""
    r = dist.get_rank(group)
    to_global = (lambda x: dist.get_global_rank(group, x)) if group is not None else (lambda x: x)
    if r == src:
        dist.send(tensor.contiguous(), to_global(dst), group=group)
    elif r == dst:
        dist.recv(tensor, to_global(src), group=group)
    return tensor


def ring_all_gather(tensor: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenate every rank's ``tensor`` along dim 0 (N-1 ring steps)."""
    n, r, nxt, prv = _ring(group)
    tensor = tensor.contiguous()
    if n == 1:
        return tensor.clone()
    chunks: List[Optional[torch.Tensor]] = [None] * n
    chunks[r] = tensor
    cur = tensor
    for step in range(n - 1):
        recv = torch.empty_like(tensor)
        _sendrecv(cur, recv, nxt, prv, group, r)
        chunks[(r - step - 1) % n] = recv
        cur = recv
    return torch.cat(chunks, dim=0)


def ring_reduce_scatter(chunks: List[torch.Tensor], group=None) -> torch.Tensor:
    """``chunks`` = N equal tensors; returns sum over ranks of chunk[rank] (N-1 ring steps)."""
    n, r, nxt, prv = _ring(group)
    assert len(chunks) == n, f"need {n} chunks, got {len(chunks)}"
    if n == 1:
        return chunks[0].clone()
    acc = [c.contiguous().clone() for c in chunks]
    # step s: send partial of chunk (r - s - 1), receive and add partial of chunk (r - s - 2);
    # after N-1 steps the fully reduced chunk that lands here is chunk r
    for step in range(n - 1):
        send_idx = (r - step - 1) % n
        recv_idx = (r - step - 2) % n
        recv = torch.empty_like(acc[recv_idx])
        _sendrecv(acc[send_idx], recv, nxt, prv, group, r)
        acc[recv_idx] += recv
    return acc[r]


def ring_all_reduce(tensor: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over ranks, in place: reduce-scatter phase then all-gather phase, 2(N-1) steps."""
    n, r, nxt, prv = _ring(group)
    if n == 1:
        return tensor
    flat = tensor.contiguous().view(-1)
    numel = flat.numel()
    per = (numel + n - 1) // n
    padded = torch.zeros(per * n, dtype=flat.dtype, device=flat.device)
    padded[:numel] = flat
    parts = list(padded.view(n, per).unbind(0))
    for step in range(n - 1):                       # reduce-scatter: chunk (r+1) ends complete on rank r
        send_idx = (r - step) % n
        recv_idx = (r - step - 1) % n
        recv = torch.empty_like(parts[recv_idx])
        _sendrecv(parts[send_idx].contiguous(), recv, nxt, prv, group, r)
        parts[recv_idx] += recv
    for step in range(n - 1):                       # all-gather of the completed chunks
        send_idx = (r - step + 1) % n
        recv_idx = (r - step) % n
        recv = torch.empty_like(parts[recv_idx])
        _sendrecv(parts[send_idx].contiguous(), recv, nxt, prv, group, r)
        parts[recv_idx].copy_(recv)
    tensor.copy_(padded[:numel].view_as(tensor))
    return tensor
