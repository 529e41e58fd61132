"""ctypes binding of the in-tree CUDA library (``lightron_b200/csrc/liblightron_b200.so``).

The library is plain ``extern "C"``: every entry point takes raw device pointers, sizes and a
``cudaStream_t`` and returns 0 or a negative error code, so it builds in seconds with nvcc alone
and does not depend on the torch C++ ABI.  On a machine with a GPU a missing library is an error
(``require()``), never a silent fallback to library kernels.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int64, c_float, c_void_p
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_LIB_ERR: Optional[str] = None
LIB_NAME = "liblightron_b200.so"


def lib_path() -> str:
    override = os.environ.get("LIGHTRON_B200_LIB")           # e.g. a build with extra instrumentation
    if override:
        return override
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", LIB_NAME)


_P, _I, _L, _F = c_void_p, c_int, c_int64, c_float

# name -> argtypes (all return int)
_SIGNATURES = {
    "lb_last_error": [],
    "lb_sm_count": [],
    "lb_set_flag_wait_ns": [ctypes.c_ulonglong],
    "lb_device_status": [_P],
    "lb_rmsnorm_fwd": [_P, _P, _P, _P, _P, _P, _I, _I, _F, _P],
    "lb_rmsnorm_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "lb_rmsnorm_bwd_blocks": [_I, _I],
    "lb_rope": [_P, _P, _P, _P, _I, _I, _I, _I, _L, _I, _P],
    "lb_swiglu_fwd": [_P, _P, _I, _I, _L, _P],
    "lb_swiglu_bwd": [_P, _P, _P, _I, _I, _L, _P],
    "lb_embedding_fwd": [_P, _P, _P, _I, _I, _I, _I, _P],
    "lb_embedding_bwd": [_P, _P, _P, _I, _I, _I, _I, _P],
    "lb_ce_stats": [_P, _P, _P, _P, _P, _I, _I, _L, _I, _P],
    "lb_ce_grad": [_P, _P, _P, _P, _P, _I, _I, _L, _I, _F, _I, _P],
    "lb_adamw": [_P, _P, _P, _P, _P, _L, _F, _F, _F, _F, _F, _F, _F, _F, _I, _P],
    "lb_sumsq": [_P, _L, _P, _I, _P],
    "lb_add_inplace": [_P, _P, _L, _P],
    "lb_gemm_bf16": [_P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _I, _I, _P],
    "lb_gemm_grouped": [_I] + [_P] * 13,
    "lb_gemm_grouped_epi": [_I] + [_P] * 17,
    "lb_peer_copy": [_P, _P, _L, _I, _I, _P],
    "lb_peer_copy_flagged": [_P, _P, _L, _I, _I, _L, _P, _P],
    "lb_embed_tp_fwd": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, ctypes.c_uint, _P],
    "lb_embed_tp_bwd": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, ctypes.c_uint, _P],
    "lb_gemm_grouped_status": [_P],
    "lb_gemm_grouped_cached": [],
    "lb_gemm_grouped_plan": [_I, _P, _P, _P, _I, _P],
    "lb_gemm_ag": [_P, _P, _I, _I, _I, _L, _L, _I, _I, _I, _P, _L, _P, _P, ctypes.c_uint, _I, _P],
    "lb_gemm_rs": [_P, _P, _I, _I, _I, _L, _L, _I, _I, _I, _P, _P, ctypes.c_uint, _P, _L, _P],
    "lb_moe_status": [_P],
    "lb_moe_router_blocks": [_I],
    "lb_moe_push_ctas": [_I],
    "lb_moe_router": [_P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P],
    "lb_moe_plan": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _I, ctypes.c_uint, _P],
    "lb_moe_push": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P],
    "lb_moe_pull": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, ctypes.c_uint, _P],
    "lb_moe_router_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "lb_gemm_ragged": [_P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _P, ctypes.c_uint, _P],
    "lb_gemm_ragged_wgrad": [_P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _P],
    "lb_swiglu_fwd_dev": [_P, _P, _I, _I, _L, _P, _P],
    "lb_swiglu_bwd_dev": [_P, _P, _P, _I, _I, _L, _P, _P],
    "lb_coll_status": [_P],
    "lb_ulysses_a2a": [_I, _P, _L, _L, _L, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, ctypes.c_uint, _P],
    "lb_cp_dkv_reduce": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, ctypes.c_uint, _P],
    "lb_gather_into": [_P, _P, _P, _P, _L, _I, _I, _I, ctypes.c_uint, _P],
    "lb_slot_release": [_P, _I, _I, ctypes.c_uint, _P],
    "lb_fsdp_rs_adamw": [_P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _I, _I, ctypes.c_uint, _F, _F, _F, _F, _F, _F, _F, _F, _I, _I, _I, _P],
    "lb_collective": [_I, _P, _P, _P, _P, _L, _L, _I, _I, _I, _I, ctypes.c_uint, _P],
    "lb_all_reduce_nvls": [_P, _P, _P, _P, _P, _L, _L, _I, _I, _I, _I, ctypes.c_uint, _P],
    "lb_dp_status": [_P],
    "lb_dp_adamw": [_P, _P, _P, _P, _P, _P, _P, _L, _L, _I, _I, ctypes.c_uint, _F, _F, _F, _F, _F, _F, _F, _F, _I, _P],
    "lb_flash_fwd": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _F, _I, _P],
    "lb_flash_fwd_tc": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _F, _I, _P],
    "lb_flash_status": [_P],
    "lb_flash_fwd_cp_mover_warps": [],
    "lb_flash_fwd_cp": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _L, _L, _F, _I, _P, ctypes.c_uint, _I, _P, _P,
                        _L, _L, _I, _I, _P, _P, _P, _I, _P],
    "lb_flash_bwd_cp": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                        _L, _L, _L, _L, _L, _L, _L, _L, _F, _I, _P],
    "lb_flash_bwd_status": [_P],
    "lb_flash_bwd_tc": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                        _L, _L, _L, _L, _L, _L, _L, _L, _F, _I, _P],
    "lb_flash_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                     _L, _L, _L, _L, _L, _L, _L, _L, _F, _I, _P],
}


def _load() -> Optional[ctypes.CDLL]:
    global _LIB, _LIB_ERR
    if _LIB is not None or _LIB_ERR is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        _LIB_ERR = f"{path} not built (run: python -m lightron_b200.csrc.build)"
        return None
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:  # pragma: no cover
        _LIB_ERR = f"cannot load {path}: {e}"
        return None
    for name, args in _SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = c_int
    _LIB = lib
    wait_ms = os.environ.get("LIGHTRON_FLAG_WAIT_MS")     # limit of every device-side wait for a peer
    if wait_ms and hasattr(lib, "lb_set_flag_wait_ns"):
        lib.lb_set_flag_wait_ns(int(float(wait_ms) * 1e6))
    return _LIB


def available() -> bool:
    """True when CUDA kernels can run: a GPU is present and the library loads."""
    return torch.cuda.is_available() and _load() is not None


def require() -> ctypes.CDLL:
    lib = _load()
    if lib is None:
        raise RuntimeError(f"lightron_b200 native kernels unavailable: {_LIB_ERR}")
    return lib


def use_native(t: torch.Tensor) -> bool:
    """CUDA bf16 tensors take the native path; anything else the PyTorch oracle path.
    On a GPU box the library must be present (loud failure instead of a silent fallback)."""
    if not t.is_cuda or t.dtype != torch.bfloat16:
        return False
    require()
    return True


def sm_count() -> int:
    """SMs of the current device (what the persistent kernels size their grids with)."""
    return int(require().lb_sm_count())


def set_flag_wait_ns(ns: int) -> None:
    """Wall-time limit after which a kernel that waits for a peer's flag gives up and reports through
    its status word (default 20 s; tests of the give-up path use a few milliseconds)."""
    rc = require().lb_set_flag_wait_ns(int(ns))
    if rc != 0:
        raise NativeError(f"lb_set_flag_wait_ns({ns}) failed: {rc}")


def measured_peaks() -> dict:
    """``MEASURED_PEAKS.json`` at the repository root when present (roofline denominators measured on
    the machine: ``hbm_gbs``, ``bf16_tflops``, ``bf16_tflops_sustained``), else the nominal figures."""
    import json
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    except Exception:
        return {"hbm_gbs": 7700.0, "bf16_tflops": 2250.0, "bf16_tflops_sustained": 2250.0, "source": "nominal"}


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


class NativeError(RuntimeError):
    pass


_ERRORS = {-1: "invalid argument", -2: "CUDA launch error", -3: "unsupported shape", -4: "driver entry point missing",
           -5: "tensor map encode failed", -6: "size exceeds static scratch capacity"}

_LAUNCHES = 0


def launch_count() -> int:
    """Number of native kernel entry points invoked so far in this process."""
    return _LAUNCHES


def call(name: str, *args) -> None:
    global _LAUNCHES
    lib = require()
    rc = getattr(lib, name)(*args)
    _LAUNCHES += 1
    if rc != 0:
        raise NativeError(f"{name} failed: {_ERRORS.get(rc, rc)} (cuda error {lib.lb_last_error()})")


_STATUS_READERS = (("lb_device_status", "GEMM / fused collective GEMM"), ("lb_gemm_grouped_status", "grouped GEMM"),
                   ("lb_flash_status", "attention forward"), ("lb_flash_bwd_status", "attention backward"),
                   ("lb_dp_status", "data-parallel optimizer kernel"),
                   ("lb_moe_status", "expert-parallel routing / dispatch / combine"),
                   ("lb_coll_status", "stand-alone peer-memory collective"))


def device_status() -> dict:
    """Status words of every kernel family that has bounded waits: ``{family: (code, where)}`` for the
    families whose wait ran out since the last read (reading clears them; synchronises the device)."""
    lib = require()
    out = {}
    buf = (ctypes.c_uint * 4)()
    for sym, family in _STATUS_READERS:
        getattr(lib, sym)(ctypes.cast(buf, ctypes.c_void_p))
        if buf[0]:
            out[family] = (int(buf[0]), int(buf[1]))
        if sym == "lb_moe_status" and buf[2]:
            MOE_DROPPED["events"] += int(buf[2])
            MOE_DROPPED["max_rows"] = max(MOE_DROPPED["max_rows"], int(buf[3]))
    return out


# Copies of tokens that expert-parallel routing dropped because an expert's rows exceeded the capacity of
# the exchange buffers (``model.moe_capacity_factor``): not an error, but worth a line in the log.
MOE_DROPPED = {"events": 0, "max_rows": 0}


def take_moe_dropped() -> dict:
    """Counts gathered by the last ``device_status`` calls, reset on read."""
    d = dict(MOE_DROPPED)
    MOE_DROPPED["events"], MOE_DROPPED["max_rows"] = 0, 0
    return d


def raise_on_device_status() -> None:
    """Turn a bounded wait that ran out inside a kernel (a peer that never arrived, a lost barrier)
    into a Python error at the next host synchronisation point instead of silently wrong numbers."""
    bad = device_status()
    if bad:
        raise RuntimeError("device-side wait ran out: " + ", ".join(f"{k} (code {c}, where {w})" for k, (c, w) in bad.items()))
