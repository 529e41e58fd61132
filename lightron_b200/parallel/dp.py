"""Replicated data parallelism (DDP style).

API parity with the reference's ``parallel/parallel_dp.py:7-41`` (``DataParallel(module)``: a
post-accumulate-grad hook per parameter that all-reduces and divides by the DP size).  Differences:
gradients are reduced in flat buckets (one collective per ~25 MB instead of one per tensor), the
reduction of a bucket starts as soon as its last gradient is ready and runs on a side stream on
GPUs, and ``no_sync()`` / ``require_backward_grad_sync`` suppress it for all but the last
micro-batch (the reference reduces on every backward).  The trainer does not use this class: its
default engine is ``optim.DistributedAdamW`` (reduce-scatter + sharded optimizer state).
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import mesh as _mesh
from . import comm


class DataParallel(nn.Module):
    def __init__(self, module: nn.Module, group="auto", bucket_mb: float = 25.0):
        super().__init__()
        self.module = module
        self.group = _mesh.get_dp_group() if group == "auto" else group
        self.dp_size = comm.group_size(self.group)
        self.require_backward_grad_sync = True
        self.buckets: List[List[nn.Parameter]] = []
        self._pending: List[int] = []
        self._work = []
        self._stream: Optional[torch.cuda.Stream] = None
        if self.dp_size > 1:
            cap = int(bucket_mb * (1 << 20))
            cur, size = [], 0
            for p in reversed([p for p in module.parameters() if p.requires_grad]):   # backward order
                cur.append(p)
                size += p.numel() * p.element_size()
                if size >= cap:
                    self.buckets.append(cur)
                    cur, size = [], 0
            if cur:
                self.buckets.append(cur)
            for bi, b in enumerate(self.buckets):
                for p in b:
                    p.register_post_accumulate_grad_hook(self._make_hook(bi))
            self._pending = [len(b) for b in self.buckets]
            if next(module.parameters()).is_cuda:
                self._stream = torch.cuda.Stream()

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)

    @contextmanager
    def no_sync(self):
        old = self.require_backward_grad_sync
        self.require_backward_grad_sync = False
        try:
            yield
        finally:
            self.require_backward_grad_sync = old

    def _make_hook(self, bi: int):
        def hook(_p):
            if not self.require_backward_grad_sync:
                return
            self._pending[bi] -= 1
            if self._pending[bi] == 0:
                self._pending[bi] = len(self.buckets[bi])
                self._reduce(bi)
        return hook

    def _reduce(self, bi: int) -> None:
        params = [p for p in self.buckets[bi] if p.grad is not None]
        if not params:
            return

        def run():
            flat = torch.cat([p.grad.reshape(-1) for p in params])
            dist.all_reduce(flat, group=self.group)
            flat.div_(self.dp_size)
            off = 0
            for p in params:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
                off += p.numel()

        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                run()
        else:
            run()

    def finish_grad_sync(self) -> None:
        """Wait for outstanding reductions (call before optimizer.step())."""
        if self._stream is not None:
            torch.cuda.current_stream().wait_stream(self._stream)
