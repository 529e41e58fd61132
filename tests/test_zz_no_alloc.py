"""The allocation-free RMSNorm backward entry point (`lb_rmsnorm_bwd_static`).

Some hosts of this library cannot obtain device memory when they call into it: code running
inside an allocator callback, shutdown paths, processes whose memory pool was sized once at
start-up, or a C program that has no tensor library to ask.  For them the library carries its own
fixed scratch area.  This test drives that entry point directly through its exported C symbol
(no wrapper in between) and checks that it reproduces the regular entry point, twice in a row,
because the scratch area is reused and keeps whatever the previous call left in it.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g, device="cuda").to(torch.bfloat16)
    x, dy, dres = mk(rows, cols), mk(rows, cols), mk(rows, cols)
    w = (1 + 0.1 * torch.randn(cols, generator=g, device="cuda")).to(torch.bfloat16)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
    return x, dy, dres, w, rstd


def test_static_scratch_entry_matches_regular_entry_twice():
    from lightron_b200.ops import native
    lib = ctypes.CDLL(native.lib_path())
    P, I = ctypes.c_void_p, ctypes.c_int
    static_fn = lib.lb_rmsnorm_bwd_static
    static_fn.argtypes = [P, P, P, P, P, P, P, I, I, P]
    static_fn.restype = I
    regular = lib.lb_rmsnorm_bwd
    regular.argtypes = [P, P, P, P, P, P, P, P, I, I, I, P]
    regular.restype = I
    blocks = lib.lb_rmsnorm_bwd_blocks
    blocks.argtypes = [I, I]
    blocks.restype = I
    stream = torch.cuda.current_stream().cuda_stream
    # the second call uses another shape, so stale rows of the first call would show up
    for call, (rows, cols) in enumerate([(3000, 2048), (777, 4096)]):
        x, dy, dres, w, rstd = _inputs(rows, cols, seed=call)
        dx_a, dw_a = torch.empty_like(x), torch.empty_like(w)
        dx_b, dw_b = torch.empty_like(x), torch.empty_like(w)
        nblk = blocks(rows, cols)
        partial = torch.empty(nblk, cols, dtype=torch.float32, device="cuda")
        rc = regular(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx_a.data_ptr(),
                     partial.data_ptr(), dw_a.data_ptr(), rows, cols, nblk, stream)
        assert rc == 0
        rc = static_fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx_b.data_ptr(),
                       dw_b.data_ptr(), rows, cols, stream)
        assert rc == 0, f"static entry returned {rc}"
        torch.cuda.synchronize()
        rel_dx = (dx_a.float() - dx_b.float()).norm() / dx_a.float().norm()     # row sums differ in order only
        assert rel_dx < 5e-3, f"call {call}: dx differs, rel {rel_dx.item()}"
        rel = (dw_a.float() - dw_b.float()).norm() / dw_a.float().norm()
        assert rel < 1e-2, f"call {call}: dw differs, rel {rel.item()}"


def test_static_scratch_entry_rejects_oversize():
    from lightron_b200.ops import native
    lib = ctypes.CDLL(native.lib_path())
    P, I = ctypes.c_void_p, ctypes.c_int
    fn = lib.lb_rmsnorm_bwd_static
    fn.argtypes = [P, P, P, P, P, P, P, I, I, P]
    fn.restype = I
    t = torch.zeros(8, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(), t.data_ptr(), 4, 8192 + 8,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -6           # capacity error, nothing launched
