"""Host-side logic around the grouped GEMM: the static schedule, the deferred weight-gradient queue
and the segment-wise linear, all without a GPU."""
import ctypes
import os

import pytest
import torch

from lightron_b200.ops import functional as OF, native


def _plan(shapes, sms=148):
    lib = native._load()
    if lib is None:
        pytest.skip("native library not built")
    n = len(shapes)
    IA = ctypes.c_int * n
    M, N, K = IA(*[s[0] for s in shapes]), IA(*[s[1] for s in shapes]), IA(*[s[2] for s in shapes])
    out = (ctypes.c_longlong * 3)()
    assert lib.lb_gemm_grouped_plan(n, M, N, K, sms, out) == 0
    busiest, work, ctas = out[0], out[1], out[2]
    return busiest * ctas / work, ctas


def test_schedule_balances_weight_gradient_with_data_gradient():
    T = 16384
    alone, _ = _plan([(2560, 2048, T)])                      # 160 tiles on 148 SMs: second wave 8 % full
    paired, ctas = _plan([(2560, 2048, T), (T, 2048, 2560)])
    assert alone > 1.8 and paired < 1.06 and ctas == 148
    # the queued weight gradients of a tensor-parallel layer (TP2 shapes of the 1.1B model)
    assert _plan([(2048, 2816, T), (5632, 2048, T)])[0] < 1.15
    assert _plan([(2048, 1024, T), (1280, 2048, T)])[0] < 1.02
    # fewer tiles than SMs: one tile per CTA
    imb, ctas = _plan([(256, 512, 4096)])
    assert ctas == 4 and imb == 1.0


def test_schedule_rejects_bad_arguments():
    lib = native._load()
    if lib is None:
        pytest.skip("native library not built")
    IA = ctypes.c_int * 1
    out = (ctypes.c_longlong * 3)()
    assert lib.lb_gemm_grouped_plan(1, IA(0), IA(8), IA(8), 148, out) != 0
    assert lib.lb_gemm_grouped_plan(9, IA(8), IA(8), IA(8), 148, out) != 0


def _fake_gemm_grouped(problems):
    outs = []
    for a, b, a_mn, b_mn, out, acc in problems:
        A = a.t() if a_mn else a
        Bm = b if b_mn else b.t()
        r = A.float() @ Bm.float()
        if out is None:
            out = torch.empty(r.shape, dtype=a.dtype)
        out.copy_((out.float() + r if acc else r).to(out.dtype))
        outs.append(out)
    return outs


class _DeferringLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        ctx.params = (w,)
        return x @ w.t()

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        assert OF.direct_wgrad_ok(ctx.params)
        OF.defer_wgrad(dy.contiguous(), x, ctx.params)
        return dy @ w, None


def test_deferred_weight_gradients_flush_once_at_end_of_backward(monkeypatch):
    monkeypatch.setattr(OF, "gemm_grouped", _fake_gemm_grouped)
    launches = []
    real = OF.gemm_grouped
    monkeypatch.setattr(OF, "gemm_grouped", lambda probs: (launches.append(len(probs)), real(probs))[1])
    torch.manual_seed(0)
    arena = torch.zeros(3 * 16 * 16)
    ws, fired = [], []
    for i in range(3):
        w = torch.nn.Parameter(torch.randn(16, 16) * 0.3)
        w.grad = arena[i * 256:(i + 1) * 256].view(16, 16)
        w._lb_direct_grad = True
        w._lb_grad_hooks = (lambda p, i=i: fired.append((i, bool(getattr(p, "_lb_wgrad_pending", False)))),)
        ws.append(w)
    x = torch.randn(5, 16, requires_grad=True)
    h = x
    for w in ws:                                        # every weight is used twice per forward
        h = _DeferringLinear.apply(h, w) + 0.5 * _DeferringLinear.apply(h, w)
    h.sum().backward()
    assert launches == [6]                              # six queued products, one grouped launch
    assert sorted(i for i, _ in fired) == [0, 0, 1, 1, 2, 2] and not any(p for _, p in fired)
    assert not OF._WQ and all(not w._lb_wgrad_pending for w in ws)
    ws2 = [w.detach().clone().requires_grad_(True) for w in ws]
    x2 = x.detach().clone().requires_grad_(True)
    h2 = x2
    for w in ws2:
        h2 = h2 @ w.t() + 0.5 * (h2 @ w.t())
    h2.sum().backward()
    for w, w2 in zip(ws, ws2):
        assert torch.allclose(w.grad, w2.grad, atol=1e-4, rtol=1e-4)
    assert torch.allclose(x.grad, x2.grad, atol=1e-4, rtol=1e-4)


def test_grouped_linear_segments_match_per_segment_math():
    torch.manual_seed(1)
    x = torch.randn(11, 16, requires_grad=True)
    groups = [(torch.randn(8, 16, requires_grad=True), torch.randn(8, 16, requires_grad=True)) for _ in range(3)]
    counts = [4, 0, 5]                                  # two rows are beyond every segment
    y = OF.grouped_linear(x, counts, groups)
    assert y.shape == (11, 16) and y[9:].abs().max().item() == 0
    want0 = torch.cat([x[:4] @ groups[0][0].t(), x[:4] @ groups[0][1].t()], dim=1)
    want2 = torch.cat([x[4:9] @ groups[2][0].t(), x[4:9] @ groups[2][1].t()], dim=1)
    assert torch.allclose(y[:4], want0, atol=1e-5) and torch.allclose(y[4:9], want2, atol=1e-5)
    y.square().sum().backward()
    assert groups[1][0].grad is None or groups[1][0].grad.abs().max().item() == 0
    assert x.grad[9:].abs().max().item() == 0 and x.grad[:9].abs().max().item() > 0


def test_bucket_hook_counts_each_parameter_once_and_skips_pending_or_unsynced():
    from lightron_b200 import mesh
    from lightron_b200.config import ModelArgs
    from lightron_b200.models import LightronTransformer, init_weights
    from lightron_b200.optim import DistributedAdamW
    mesh.set_context(None)
    args = ModelArgs(dim=32, n_layers=1, n_heads=2, n_kv_heads=2, vocab_size=64, intermediate_size=64, max_seq_len=16)
    m = LightronTransformer(args, dtype=torch.float32, device=torch.device("cpu"))
    init_weights(m, 0)
    opt = DistributedAdamW(m, lr=1e-3)
    assert opt.grad_shard.data_ptr() == opt.flat_grads.data_ptr()        # no replicas: shards alias the arenas
    b = opt.buckets[0]
    launched = []
    opt._launch_reduce = lambda bb, async_op: launched.append(bb)
    hook = opt._make_hook(b)
    p0, p1 = opt.params[0], opt.params[1]
    b.pending, b.seen = 2, set()
    hook(p0); hook(p0)                                   # by hand and again by autograd: one count
    assert b.pending == 1 and not launched
    p1._lb_wgrad_pending = True
    hook(p1)                                             # its weight gradient is still queued
    assert b.pending == 1
    p1._lb_wgrad_pending = False
    with opt.no_sync():
        hook(p1)                                         # micro-batch without gradient sync
    assert b.pending == 1
    hook(p1)
    assert b.pending == 0 and launched == [b]
    opt._reset_buckets()
    assert b.pending == b.n_params and not b.seen


_SAN_SCRIPT = r'''
import ctypes, random, sys
lib = ctypes.CDLL(sys.argv[1])
random.seed(0)
# host-only entry points (no CUDA call): the static schedule of the grouped GEMM for many shape sets
for trial in range(200):
    n = random.randint(1, 8)
    IA = ctypes.c_int * n
    M = IA(*[random.choice([8, 128, 1000, 4096, 16384]) for _ in range(n)])
    N = IA(*[random.choice([8, 264, 2048, 11264]) for _ in range(n)])
    K = IA(*[random.choice([8, 200, 2048, 16384]) for _ in range(n)])
    out = (ctypes.c_longlong * 3)()
    rc = lib.lb_gemm_grouped_plan(n, M, N, K, random.choice([1, 7, 148]), out)
    assert rc == 0 and out[0] > 0 and out[1] >= out[0] and out[2] >= 1, (rc, list(out))
IA1 = ctypes.c_int * 1
out = (ctypes.c_longlong * 3)()
assert lib.lb_gemm_grouped_plan(0, IA1(8), IA1(8), IA1(8), 148, out) != 0
assert lib.lb_gemm_grouped_plan(1, IA1(-5), IA1(8), IA1(8), 148, out) != 0
lib.lb_set_flag_wait_ns.argtypes = [ctypes.c_ulonglong]
assert lib.lb_set_flag_wait_ns(5_000_000) == 0
assert lib.lb_gemm_grouped_cached() == 0
print("SANITIZED_HOST_OK")
'''


def test_host_code_under_address_and_ub_sanitizers(tmp_path):
    """The C++ host side of the library (argument checks, the grouped GEMM's schedule builder) built with
    -fsanitize=address,undefined and driven without a GPU: any out-of-bounds access, use after free or
    undefined arithmetic in it aborts the child process."""
    import shutil
    import subprocess
    import sys
    from lightron_b200.csrc import build as B
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    if not os.path.exists(nvcc) or shutil.which("gcc") is None:
        pytest.skip("needs nvcc and gcc")
    asan = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not os.path.isabs(asan) or not os.path.exists(asan):
        pytest.skip("libasan not installed")
    lib = B.build_sanitized(str(tmp_path / "liblightron_b200_asan.so"))
    script = tmp_path / "san.py"
    script.write_text(_SAN_SCRIPT)
    env = dict(os.environ, LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:protect_shadow_gap=0:abort_on_error=1",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([sys.executable, str(script), lib], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "SANITIZED_HOST_OK" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]
