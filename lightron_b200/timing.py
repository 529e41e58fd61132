"""Device-side step timing (CUDA events, MAX over ranks) with a wall-clock fallback on CPU.

The reference measures throughput as tokens / wall-clock since the loop started
(trainer.py:285,316-328) and times only its ring-attention demo with CUDA events
(parallel/communication/ring_attention.py:186-196)."""
from __future__ import annotations

import time
from typing import List

import torch
import torch.distributed as dist


class StepTimer:
    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        self.device = device
        self._pairs: List = []
        self._t0 = None
        self._wall: List[float] = []

    def start(self):
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._t0 = e
        else:
            self._t0 = time.perf_counter()

    def stop(self):
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pairs.append((self._t0, e))
        else:
            self._wall.append((time.perf_counter() - self._t0) * 1e3)

    def reset(self):
        self._pairs, self._wall = [], []

    def mean_ms(self) -> float:
        if self.cuda:
            if not self._pairs:
                return 0.0
            self._pairs[-1][1].synchronize()
            return sum(a.elapsed_time(b) for a, b in self._pairs) / len(self._pairs)
        return sum(self._wall) / max(len(self._wall), 1)

    def mean_ms_max_over_ranks(self) -> float:
        ms = self.mean_ms()
        if dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms
