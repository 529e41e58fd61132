"""Numerics of every CUDA kernel against a plain PyTorch fp32 restatement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _rand(*shape, scale=1.0, dtype=torch.bfloat16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _gemm_status():
    import ctypes
    from lightron_b200.ops import native
    buf = (ctypes.c_uint * 4)()
    native.require().lb_device_status(ctypes.cast(buf, ctypes.c_void_p))
    buf2 = (ctypes.c_uint * 4)()
    native.require().lb_gemm_grouped_status(ctypes.cast(buf2, ctypes.c_void_p))
    return [a | b for a, b in zip(buf, buf2)]


def _rel_err(got, want):
    return ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-12)).item()


# ---- GEMM -------------------------------------------------------------------------------------


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)],
                         ids=["kk", "kmn", "mnmn", "mnk"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 264, 200), (1000, 1032, 520), (4096, 2560, 2048)])
@pytest.mark.parametrize("legacy", [False, True], ids=["grouped1", "plain"])
def test_gemm_all_majors(M, N, K, a_mn, b_mn, legacy):
    from lightron_b200.ops import functional as OF
    if a_mn and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0")
    a = _rand(M, K, seed=1)
    b = _rand(N, K, seed=2)
    want = a.float() @ b.float().t()
    a_arg = a.t().contiguous() if a_mn else a
    b_arg = b.t().contiguous() if b_mn else b
    got = OF.gemm(a_arg, b_arg, a_mn=a_mn, b_mn=b_mn, legacy=legacy)
    torch.cuda.synchronize()
    st = _gemm_status()
    assert st[0] == 0, f"device status {st}"
    err = _rel_err(got, want)
    assert err < 5e-3, f"rel err {err} (a_mn={a_mn}, b_mn={b_mn}, {M}x{N}x{K}); max abs {(got.float()-want).abs().max().item()}"


def test_gemm_grouped_mixed_problems():
    """Four problems of different size and operand majors in one launch, one of them accumulating
    into its output; every result against fp32 matmul."""
    import ctypes
    from lightron_b200.ops import functional as OF, native
    specs = [(2048, 1536, 512, False, True), (520, 264, 4096, True, True), (128, 256, 64, False, False),
             (1000, 1032, 520, True, False)]
    probs, wants = [], []
    for i, (M, N, K, a_mn, b_mn) in enumerate(specs):
        a, b = _rand(M, K, seed=10 + i), _rand(N, K, seed=20 + i)
        want = a.float() @ b.float().t()
        out, acc = None, False
        if i == 1:
            out, acc = _rand(M, N, seed=30), True
            want = want + out.float()
        probs.append((a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b, a_mn, b_mn, out, acc))
        wants.append(want)
    for _ in range(2):                                   # second call reuses the cached schedule
        if probs[1][4] is not None:
            probs[1] = probs[1][:4] + (_rand(520, 264, seed=30), True)
        outs = OF.gemm_grouped(probs)
        torch.cuda.synchronize()
        buf = (ctypes.c_uint * 4)()
        native.require().lb_gemm_grouped_status(ctypes.cast(buf, ctypes.c_void_p))
        assert buf[0] == 0, f"device status {list(buf)}"
        for got, want in zip(outs, wants):
            assert _rel_err(got, want) < 5e-3


def test_linear_backward_grouped_matches_separate(monkeypatch):
    from lightron_b200.ops import functional as OF
    x = _rand(1024, 512, seed=1).requires_grad_(True)
    w = _rand(776, 512, seed=2, scale=0.05).requires_grad_(True)
    dy = _rand(1024, 776, seed=3)
    grads = []
    for flag in (True, False):
        monkeypatch.setattr(OF, "_GROUP_BWD", flag)
        x.grad = w.grad = None
        OF.linear(x, w).backward(dy)
        grads.append((x.grad.clone(), w.grad.clone()))
    assert _rel_err(grads[0][0], grads[1][0]) < 1e-3 and _rel_err(grads[0][1], grads[1][1]) < 1e-3
    assert _rel_err(grads[0][0], dy.float() @ w.detach().float()) < 5e-3
    assert _rel_err(grads[0][1], dy.float().t() @ x.detach().float()) < 5e-3


def test_gemm_strided_operands_and_output():
    from lightron_b200.ops import functional as OF
    big = _rand(512, 1024, seed=3)
    a = big[:, 256:768]                      # row stride 1024, K = 512
    w = _rand(384, 512, seed=4)
    out_big = torch.zeros(512, 1024, dtype=torch.bfloat16, device="cuda")
    out = out_big[:, 128:512]
    OF.gemm(a, w, out=out)
    torch.cuda.synchronize()
    want = a.float() @ w.float().t()
    assert _rel_err(out, want) < 5e-3
    assert out_big[:, :128].abs().max().item() == 0 and out_big[:, 512:].abs().max().item() == 0


def test_linear_autograd_fused_weights():
    from lightron_b200.ops import functional as OF
    T, K = 512, 256
    x = _rand(T, K, seed=5).requires_grad_(True)
    flat = _rand(3 * 128 * K, scale=0.05, seed=6)
    ws = [flat[i * 128 * K:(i + 1) * 128 * K].view(128, K).requires_grad_(True) for i in range(3)]
    assert OF._rows_adjacent(ws)
    y = OF.linear(x, *ws)
    dy = _rand(T, 384, seed=7)
    y.backward(dy)
    xf = x.detach().float().requires_grad_(True)
    wf = [w.detach().float().requires_grad_(True) for w in ws]
    yf = torch.cat([xf @ w.t() for w in wf], dim=1)
    yf.backward(dy.float())
    assert _rel_err(y, yf) < 5e-3
    assert _rel_err(x.grad, xf.grad) < 5e-3
    for w, wr in zip(ws, wf):
        assert _rel_err(w.grad, wr.grad) < 5e-3


# ---- elementwise ------------------------------------------------------------------------------------


@pytest.mark.parametrize("rows,cols", [(64, 256), (1000, 2048), (333, 4096), (129, 768), (77, 6144), (50, 8192), (40, 264)])
def test_rmsnorm_fwd_bwd(rows, cols):
    from lightron_b200.ops import functional as OF, reference as ref
    x = _rand(rows, cols, seed=1).requires_grad_(True)
    w = (1 + 0.1 * _rand(cols, seed=2).float()).to(torch.bfloat16).requires_grad_(True)
    y = OF.rmsnorm(x, w, 1e-5)
    dy = _rand(rows, cols, seed=3)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yf = ref.rmsnorm(xf, wf, 1e-5)
    yf.backward(dy.float())
    assert _rel_err(y, yf) < 5e-3
    assert _rel_err(x.grad, xf.grad) < 1e-2
    assert _rel_err(w.grad, wf.grad) < 1e-2


def test_add_rmsnorm_fwd_bwd():
    from lightron_b200.ops import functional as OF, reference as ref
    rows, cols = 512, 2048
    x = _rand(rows, cols, seed=1).requires_grad_(True)
    r = _rand(rows, cols, seed=2).requires_grad_(True)
    w = (1 + 0.1 * _rand(cols, seed=3).float()).to(torch.bfloat16).requires_grad_(True)
    h, y = OF.add_rmsnorm(x, r, w, 1e-5)
    dh, dy = _rand(rows, cols, seed=4), _rand(rows, cols, seed=5)
    torch.autograd.backward([h, y], [dh, dy])
    xf, rf, wf = (t.detach().float().requires_grad_(True) for t in (x, r, w))
    hf = xf + rf
    yf = ref.rmsnorm(hf, wf, 1e-5)
    torch.autograd.backward([hf, yf], [dh.float(), dy.float()])
    assert _rel_err(h, hf) < 5e-3 and _rel_err(y, yf) < 5e-3
    assert _rel_err(x.grad, xf.grad) < 1e-2 and _rel_err(r.grad, rf.grad) < 1e-2
    assert _rel_err(w.grad, wf.grad) < 1e-2


@pytest.mark.parametrize("d", [32, 64, 128])
def test_rope_matches_complex_reference(d):
    from lightron_b200.ops import functional as OF, reference as ref
    B, S, h = 2, 96, 4
    x = _rand(B, S, h, d, seed=1).requires_grad_(True)
    cos, sin = ref.rope_tables(d, 128, 10000.0, device="cuda")
    pos = torch.arange(S, device="cuda").flip(0).to(torch.int32).contiguous()
    for positions in (None, pos):
        x.grad = None
        y = OF.rope(x, cos, sin, positions)
        dy = _rand(B, S, h, d, seed=2)
        y.backward(dy)
        # complex-number oracle (the reference's formulation, layers/layers.py:44-70)
        ang = torch.outer((torch.arange(S, device="cuda") if positions is None else positions).float(),
                          1.0 / (10000.0 ** (torch.arange(0, d, 2, device="cuda").float() / d)))
        fc = torch.polar(torch.ones_like(ang), ang).view(1, S, 1, d // 2)
        xf = x.detach().float().requires_grad_(True)
        yc = torch.view_as_real(torch.view_as_complex(xf.reshape(B, S, h, d // 2, 2)) * fc).flatten(3)
        yc.backward(dy.float())
        assert _rel_err(y, yc) < 5e-3
        assert _rel_err(x.grad, xf.grad) < 5e-3


def test_swiglu_fwd_bwd():
    from lightron_b200.ops import functional as OF
    rows, I = 300, 688
    gu = _rand(rows, 2 * I, seed=1).requires_grad_(True)
    y = OF.swiglu(gu)
    dy = _rand(rows, I, seed=2)
    y.backward(dy)
    gf = gu.detach().float().requires_grad_(True)
    yf = torch.nn.functional.silu(gf[:, :I]) * gf[:, I:]
    yf.backward(dy.float())
    assert _rel_err(y, yf) < 5e-3
    assert _rel_err(gu.grad, gf.grad) < 1e-2


@pytest.mark.parametrize("T,K,I", [(300, 256, 688), (1024, 512, 1408), (2048, 2048, 5632)])
def test_swiglu_mlp_fused_epilogues(T, K, I):
    """Gate | up GEMM with the activation in its epilogue, and the down projection's data gradient with
    the activation's backward in its epilogue: same bits as the three-launch path, and close to fp32."""
    from lightron_b200.ops import functional as OF
    ws = _rand(2 * I + K, max(K, I), scale=0.03, seed=3)
    w13 = ws[:2 * I, :K].contiguous()
    w1, w3 = w13[:I].requires_grad_(True), w13[I:].requires_grad_(True)
    w2 = ws[2 * I:, :I].contiguous().requires_grad_(True)
    x = _rand(T, K, seed=4).requires_grad_(True)
    dy = _rand(T, K, seed=5)
    assert OF.swiglu_mlp_ok(x, w1, w3, w2)
    y = OF.swiglu_mlp(x, w1, w3, w2)
    y.backward(dy)
    got = [y.detach().clone()] + [t.grad.clone() for t in (x, w1, w3, w2)]
    for t in (x, w1, w3, w2):
        t.grad = None
    y2 = OF.linear(OF.swiglu(OF.linear(x, w1, w3)), w2)
    y2.backward(dy)
    want = [y2.detach()] + [t.grad for t in (x, w1, w3, w2)]
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    xf, w1f, w3f, w2f = [t.detach().float().requires_grad_(True) for t in (x, w1, w3, w2)]
    yf = (torch.nn.functional.silu(xf @ w1f.t()) * (xf @ w3f.t())) @ w2f.t()
    yf.backward(dy.float())
    assert _rel_err(got[0], yf) < 1e-2
    for a, b in zip(got[1:], (xf.grad, w1f.grad, w3f.grad, w2f.grad)):
        assert _rel_err(a, b) < 2e-2
    assert _gemm_status()[0] == 0


@pytest.mark.parametrize("mode", [0, 1], ids=["stores", "bulk"])
@pytest.mark.parametrize("nbytes,ctas", [(16, 1), (16384 * 3 + 4096 + 16, 2), ((8 << 20) + 48, 16), (64 << 20, 148)])
def test_peer_copy_kernel_local(mode, nbytes, ctas):
    """The SM-issued copy the fused kernels' movers are built on (here into local memory)."""
    from lightron_b200.ops import native
    src = torch.randint(0, 255, (nbytes,), device="cuda", dtype=torch.uint8)
    dst = torch.zeros(nbytes + 64, device="cuda", dtype=torch.uint8)
    native.call("lb_peer_copy", src.data_ptr(), dst.data_ptr(), nbytes, mode, ctas, native.stream_ptr())
    torch.cuda.synchronize()
    assert torch.equal(dst[:nbytes], src)
    assert int(dst[nbytes:].sum()) == 0
    assert not native.device_status()


def test_grouped_gemm_schedule_cache_stays_bounded():
    """Callers whose shapes change from call to call must not grow the schedule cache (or device memory)
    without bound: sweeps over 150 different row counts leave at most the cache's capacity of entries behind,
    and a second sweep (every entry evicted and rebuilt) does not cost device memory."""
    from lightron_b200.ops import functional as OF, native
    lib = native.require()
    a = _rand(1208, 64, seed=1)
    b = _rand(64, 64, seed=2)
    out = torch.empty(1208, 64, device="cuda", dtype=torch.bfloat16)

    def sweep(check):
        for i, M in enumerate(range(8, 1208, 8)):                  # 150 shape sets
            OF.gemm_grouped([(a[:M], b, False, False, out[:M], False)])
            if check and i % 37 == 0:
                want = a[:M].float() @ b.float().t()
                assert _rel_err(out[:M], want) < 1e-2, M
        torch.cuda.synchronize()

    sweep(True)                                                    # also pays every one-time allocation (library handles, ...)
    assert lib.lb_gemm_grouped_cached() <= 128
    free1 = torch.cuda.mem_get_info()[0]
    sweep(False)
    assert lib.lb_gemm_grouped_cached() <= 128
    assert free1 - torch.cuda.mem_get_info()[0] < (8 << 20)
    assert _gemm_status()[0] == 0


def test_embedding_fwd_bwd_vocab_parallel():
    from lightron_b200.ops import functional as OF
    V, H, T = 1000, 256, 4096
    w = _rand(500, H, seed=1).requires_grad_(True)         # holds vocab ids [250, 750)
    tok = torch.randint(0, V, (8, T // 8), device="cuda")
    y = OF.embedding(tok, w, 250)
    dy = _rand(8, T // 8, H, seed=2)
    y.backward(dy)
    wf = w.detach().float().requires_grad_(True)
    local = tok - 250
    mask = (local < 0) | (local >= 500)
    yf = torch.nn.functional.embedding(local.clamp(0, 499), wf) * (~mask).unsqueeze(-1)
    yf.backward(dy.float())
    assert torch.equal(y.float(), yf.detach())
    assert _rel_err(w.grad, wf.grad) < 2e-2           # bf16 atomics accumulate with rounding


@pytest.mark.parametrize("T,V", [(257, 8192), (1024, 32000), (64, 1024), (33, 264)])
def test_cross_entropy_fwd_bwd(T, V):
    from lightron_b200.ops import functional as OF
    logits = _rand(T, V, scale=2.0, seed=1)
    tgt = torch.randint(0, V, (T,), device="cuda")
    lf = logits.float().requires_grad_(True)
    want = torch.nn.functional.cross_entropy(lf, tgt)
    (want * 0.5).backward()
    lg = logits.clone().requires_grad_(True)
    got = OF.cross_entropy(lg * 1.0, tgt, n_valid_total=T)
    (got * 0.5).backward()
    assert abs(got.item() - want.item()) < 2e-3 * max(1.0, abs(want.item()))
    assert _rel_err(lg.grad, lf.grad) < 2e-2


def test_adamw_matches_torch():
    from lightron_b200.ops import native
    n = 1 << 16
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").to(torch.bfloat16)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, weight_decay=0.1)
    master, m, v = p.clone(), torch.zeros_like(p), torch.zeros_like(p)
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    for step in range(1, 4):
        ref_p.grad = g.float()
        opt.step()
        native.call("lb_adamw", master.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), out.data_ptr(), n,
                    1e-2, 0.9, 0.999, 1e-8, 0.1, 1 - 0.9 ** step, 1 - 0.999 ** step, 1.0, 0, native.stream_ptr())
    torch.cuda.synchronize()
    assert torch.allclose(master, ref_p.detach(), atol=1e-5, rtol=1e-4)
    assert torch.equal(out, master.to(torch.bfloat16))


# ---- attention ------------------------------------------------------------------------------------


@pytest.mark.parametrize("d", [32, 64, 128])
@pytest.mark.parametrize("B,Sq,Sk,hq,hkv,causal", [
    (2, 128, 128, 4, 4, True), (1, 256, 256, 8, 2, True), (2, 200, 200, 4, 1, True),
    (1, 192, 320, 4, 2, False), (1, 128, 64, 2, 2, False), (1, 64, 192, 2, 1, True),
])
def test_flash_attention_fwd_bwd(B, Sq, Sk, hq, hkv, causal, d):
    from lightron_b200.ops import functional as OF, reference as ref
    q = _rand(B, Sq, hq, d, seed=1).requires_grad_(True)
    k = _rand(B, Sk, hkv, d, seed=2).requires_grad_(True)
    v = _rand(B, Sk, hkv, d, seed=3).requires_grad_(True)
    o = OF.flash_attention(q, k, v, causal)
    do = _rand(B, Sq, hq, d, seed=4)
    o.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    of = ref.attention(qf, kf, vf, causal=causal)
    of.backward(do.float())
    assert _rel_err(o, of) < 1e-2, f"fwd {_rel_err(o, of)}"
    assert _rel_err(q.grad, qf.grad) < 2e-2, f"dq {_rel_err(q.grad, qf.grad)}"
    assert _rel_err(k.grad, kf.grad) < 2e-2, f"dk {_rel_err(k.grad, kf.grad)}"
    assert _rel_err(v.grad, vf.grad) < 2e-2, f"dv {_rel_err(v.grad, vf.grad)}"


def test_rope_attention_on_fused_qkv():
    from lightron_b200.ops import functional as OF, reference as ref
    B, S, hq, hkv, d = 2, 256, 8, 2, 64
    width = (hq + 2 * hkv) * d
    base = _rand(B * S, width, seed=1)
    cos, sin = ref.rope_tables(d, S, 10000.0, device="cuda")
    x = base.clone().requires_grad_(True)
    o = OF.rope_attention_qkv(x * 1.0, cos, sin, None, B, S, hq, hkv, d)
    do = _rand(B * S, hq * d, seed=2)
    o.backward(do)
    xf = base.float().requires_grad_(True)
    of = OF.rope_attention_qkv(xf, cos, sin, None, B, S, hq, hkv, d)     # fp32 tensors take the oracle path
    of.backward(do.float())
    assert _rel_err(o, of) < 1e-2
    assert _rel_err(x.grad, xf.grad) < 2e-2


@pytest.mark.parametrize("B,S,hq,hkv,d", [(1, 2048, 8, 1, 64), (1, 8192, 8, 1, 128), (2, 1000, 8, 1, 64), (1, 777, 4, 4, 128)])
def test_flash_attention_long_sequences(B, S, hq, hkv, d):
    """Sequence lengths of the benchmark shapes (16 and 64 key blocks: the K/V and Q/dO stage rings
    wrap many times, query tiles differ by many key blocks), hq / hkv = 8, lengths that are not
    multiples of 128; forward and every gradient against the fp32 oracle."""
    from lightron_b200.ops import functional as OF, reference as ref
    q = _rand(B, S, hq, d, seed=1).requires_grad_(True)
    k = _rand(B, S, hkv, d, seed=2).requires_grad_(True)
    v = _rand(B, S, hkv, d, seed=3).requires_grad_(True)
    o = OF.flash_attention(q, k, v, True)
    do = _rand(B, S, hq, d, seed=4)
    o.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    of = ref.attention(qf, kf, vf, causal=True)
    of.backward(do.float())
    torch.cuda.synchronize()
    from lightron_b200.ops import native
    assert not native.device_status()
    assert _rel_err(o, of) < 1e-2, f"fwd {_rel_err(o, of)}"
    assert _rel_err(q.grad, qf.grad) < 2e-2, f"dq {_rel_err(q.grad, qf.grad)}"
    assert _rel_err(k.grad, kf.grad) < 2e-2, f"dk {_rel_err(k.grad, kf.grad)}"
    assert _rel_err(v.grad, vf.grad) < 2e-2, f"dv {_rel_err(v.grad, vf.grad)}"


def test_peer_wait_runs_out_and_reports():
    """A device-side wait on a peer that never arrives: with a limit of a few milliseconds the
    kernel returns, the status word is set, the host raises, and nothing was updated.  The 'peer'
    is a second rank of the data-parallel optimizer kernel that is simply never launched (its flag
    word stays 0); both ranks' arenas live on this one GPU."""
    import ctypes
    from lightron_b200.ops import native
    n = 4096
    grads = [torch.ones(n, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    params = [torch.full((n,), 3.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2)]
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    master = torch.full((n // 2,), 3.0, device="cuda")
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    arr = lambda ts: (ctypes.c_void_p * 2)(*[t.data_ptr() for t in ts])
    native.device_status()                                   # clear
    native.set_flag_wait_ns(5_000_000)                       # 5 ms
    try:
        native.call("lb_dp_adamw", arr(grads), arr(params), arr(flags), counter.data_ptr(), master.data_ptr(), m.data_ptr(),
                    v.data_ptr(), 0, n // 2, 2, 0, 1, 1e-2, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001, 1.0, 4, native.stream_ptr())
        torch.cuda.synchronize()                             # the kernel came back by itself
    finally:
        native.set_flag_wait_ns(20_000_000_000)
    assert float(master.min()) == 3.0 and float(master.max()) == 3.0          # update skipped
    assert float(m.abs().max()) == 0.0 and float(params[1].float().min()) == 3.0
    with pytest.raises(RuntimeError, match="data-parallel optimizer"):
        native.raise_on_device_status()
    assert not native.device_status()                        # reading cleared it
