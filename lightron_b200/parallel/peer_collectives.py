"""Stand-alone collectives over NVLink peer memory (``csrc/collectives.cu``): one kernel each for
all-gather, reduce-scatter, all-reduce and all-to-all of small and medium tensors, plus an
all-reduce whose sum is done inside the NVSwitch (``multimem.ld_reduce`` / ``multimem.st``).

Reference counterparts: the hand-rolled rings of ``parallel/communication/all_reduce.py:26-93``,
``ring_all_gather.py:25-58``, ``ring_reduce_scatter.py:25-68`` (N-1 ``batch_isend_irecv`` steps each)
and the ``dist.all_to_all`` of ``parallel/parallel_cp.py:71``.  ``parallel/collectives.py`` keeps the
ring algorithms as a CPU / teaching path; these are what a CUDA run uses for messages that are too
small to be worth fusing into a GEMM (loss statistics, norm-weight gradients, routing tables).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import native

_OPS = {"all_gather": 0, "all_to_all": 1, "reduce_scatter": 2, "all_reduce": 3}


class PeerComm:
    """Staging buffer + flag table of one process group in symmetric memory.

    ``max_bytes`` bounds the staged message (for all-gather / all-to-all / reduce-scatter that is the
    whole n-chunk tensor, for all-reduce the tensor itself).  ``ctas``: CTAs per collective kernel
    (also the second dimension of the flag table, so it is fixed per communicator).
    """

    def __init__(self, group, max_bytes: int = 8 << 20, ctas: int = 32, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.n = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.G = int(ctas)
        self.half = (int(max_bytes) + 4095) // 4096 * 4096
        device = device or torch.device("cuda", torch.cuda.current_device())
        flag_bytes = (2 * self.n * self.G * 4 + 4095) // 4096 * 4096
        self.flag_off = 0
        self.stage_off = flag_bytes
        self.buf = symm_mem.empty(flag_bytes + 2 * self.half, dtype=torch.uint8, device=device)
        self.buf[:flag_bytes].zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group=group)
        off = int(getattr(self.hdl, "offset", 0))
        self.ptrs = [int(p) + off for p in self.hdl.buffer_ptrs]
        mc = getattr(self.hdl, "multicast_ptr", 0) or 0
        self.mc_ptr = (int(mc) + off) if mc else 0                     # 0: no NVLS mapping on this system
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self.call = 0

    def _arr(self, off: int):
        a = (ctypes.c_void_p * self.n)()
        for r in range(self.n):
            a[r] = self.ptrs[r] + off
        return a

    def _run(self, op: str, x: torch.Tensor, out: torch.Tensor, chunk_elems: int) -> torch.Tensor:
        assert x.is_cuda and x.is_contiguous() and out.is_contiguous() and x.dtype in (torch.bfloat16, torch.float32)
        self.call += 1
        native.call("lb_collective", _OPS[op], x.data_ptr(), out.data_ptr(), self._arr(self.stage_off), self._arr(self.flag_off),
                    self.half, chunk_elems, x.element_size(), self.n, self.rank, self.G, self.call, native.stream_ptr())
        return out

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """x [m, ...] -> [n * m, ...] (rank order)."""
        out = torch.empty((self.n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        return self._run("all_gather", x.contiguous(), out, x.numel())

    def all_to_all(self, x: torch.Tensor) -> torch.Tensor:
        """x [n * m, ...]: chunk j goes to rank j; returns [n * m, ...] with chunk s from rank s."""
        assert x.shape[0] % self.n == 0
        return self._run("all_to_all", x.contiguous(), torch.empty_like(x), x.numel() // self.n)

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """x [n * m, ...] -> this rank's [m, ...] chunk of the sum over ranks (fp32 accumulation)."""
        assert x.shape[0] % self.n == 0
        out = torch.empty((x.shape[0] // self.n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        return self._run("reduce_scatter", x.contiguous(), out, x.numel() // self.n)

    def all_reduce(self, x: torch.Tensor, nvls: Optional[bool] = None) -> torch.Tensor:
        """Sum over ranks (out of place).  ``nvls``: let the switch reduce (needs a multicast mapping;
        default: use it when there is one and the tensor is at least 64 KiB)."""
        x = x.contiguous()
        out = torch.empty_like(x)
        use_nvls = (self.mc_ptr != 0 and x.numel() * x.element_size() >= (64 << 10)) if nvls is None else bool(nvls)
        if use_nvls:
            if not self.mc_ptr:
                raise RuntimeError("no NVLS multicast mapping for this group")
            self.call += 1
            native.call("lb_all_reduce_nvls", x.data_ptr(), out.data_ptr(), self._arr(self.stage_off), self.mc_ptr + self.stage_off,
                        self._arr(self.flag_off), self.half, x.numel(), x.element_size(), self.n, self.rank, self.G, self.call,
                        native.stream_ptr())
            return out
        return self._run("all_reduce", x, out, x.numel())


_COMMS: Dict[int, PeerComm] = {}


def get(group, max_bytes: int = 8 << 20) -> PeerComm:
    """The group's communicator (created collectively on first use)."""
    c = _COMMS.get(id(group))
    if c is None or c.half < max_bytes:
        c = _COMMS[id(group)] = PeerComm(group, max_bytes)
    return c
