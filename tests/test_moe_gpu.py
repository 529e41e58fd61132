"""The mixture-of-experts kernel chain (router, plan, push, ragged expert GEMMs, pull) on one GPU
against PyTorch restatements, and the whole fused feed-forward against the library-call path."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, dtype=torch.bfloat16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _rel_err(got, want):
    return ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-12)).item()


def _moe_status():
    from lightron_b200.ops import native
    buf = (ctypes.c_uint * 4)()
    native.require().lb_moe_status(ctypes.cast(buf, ctypes.c_void_p))
    return list(buf)


@pytest.mark.parametrize("T,H,E,k", [(100, 256, 8, 2), (512, 1024, 4, 1), (257, 512, 40, 3)])
def test_router_matches_torch(T, H, E, k):
    from lightron_b200.ops import native
    x, wg = _rand(T, H, seed=1), _rand(E, H, scale=0.05, seed=2)
    lib = native.require()
    nblk = lib.lb_moe_router_blocks(T)
    dev = x.device
    probs = torch.empty(T, E, device=dev)
    idx = torch.empty(T, k, dtype=torch.int32, device=dev)
    wts = torch.empty(T, k, device=dev)
    within = torch.zeros(nblk * 32, k, dtype=torch.int32, device=dev)
    hist = torch.empty(nblk, E, dtype=torch.int32, device=dev)
    psum = torch.empty(nblk, E, device=dev)
    native.call("lb_moe_router", x.data_ptr(), wg.data_ptr(), T, H, E, k, probs.data_ptr(), idx.data_ptr(), wts.data_ptr(),
                within.data_ptr(), hist.data_ptr(), psum.data_ptr(), native.stream_ptr())
    want = torch.softmax(x.float() @ wg.float().t(), dim=-1)
    assert torch.allclose(probs, want, atol=2e-5, rtol=1e-4)
    w_ref, i_ref = torch.topk(probs, k, dim=-1)                     # top-k of the kernel's own probabilities
    assert torch.allclose(wts, w_ref, atol=0, rtol=0)
    assert torch.equal(torch.gather(probs, 1, idx.long()), wts)     # an index may differ only between exact ties
    assert torch.equal(hist.sum(0).long(), torch.bincount(idx.reshape(-1).long(), minlength=E))
    assert torch.allclose(psum.sum(0), probs.sum(0), atol=1e-3, rtol=1e-5)
    # within: rank among the same expert's copies of the same 32-token block, in (token, slot) order
    flat = idx.reshape(-1).cpu()
    got = within[:T].reshape(-1).cpu()
    seen = {}
    for c in range(T * k):
        key = ((c // k) // 32, int(flat[c]))
        assert int(got[c]) == seen.get(key, 0)
        seen[key] = seen.get(key, 0) + 1


def test_ragged_gemm_matches_dense():
    """Segments of different sizes (one empty), zero padding rows, forward / data-gradient majors
    and the weight gradient, against fp32 matmuls per segment."""
    from lightron_b200.parallel import ep_fused
    LE, K, N = 4, 320, 264
    counts = [200, 0, 129, 64]
    offs, o = [], 0
    for c in counts:
        offs.append(o)
        o += (c + 127) // 128 * 128
    cap = o + 128
    seg = torch.tensor(offs + counts + [o, sum(counts)], dtype=torch.int32, device="cuda")
    A = torch.zeros(cap, K, dtype=torch.bfloat16, device="cuda")
    for e, (of, c) in enumerate(zip(offs, counts)):
        A[of:of + c] = _rand(c, K, seed=10 + e)
    W = [_rand(N, K, scale=0.1, seed=20 + e) for e in range(LE)]
    C = torch.full((cap, N), 7.0, dtype=torch.bfloat16, device="cuda")
    ep_fused._ragged(A, W, C, seg, LE, cap, N, K, False)
    for e, (of, c) in enumerate(zip(offs, counts)):
        if c:
            assert _rel_err(C[of:of + c], A[of:of + c].float() @ W[e].float().t()) < 5e-3
            pad = C[of + c:of + (c + 127) // 128 * 128]
            assert pad.numel() == 0 or float(pad.float().abs().max()) == 0.0      # zero rows in, zero rows out
    # data-gradient majors: C2 = C . W  (W stored [K_red = N, N_out = K])
    C2 = torch.empty(cap, K, dtype=torch.bfloat16, device="cuda")
    Cz = C.clone()
    Cz[o:] = 0
    ep_fused._ragged(Cz, W, C2, seg, LE, cap, K, N, True)
    for e, (of, c) in enumerate(zip(offs, counts)):
        if c:
            assert _rel_err(C2[of:of + c], Cz[of:of + c].float() @ W[e].float()) < 5e-3
    # weight gradient: G_e += dY_e^T X_e, accumulated on top of ones
    dY = torch.zeros(cap, N, dtype=torch.bfloat16, device="cuda")
    for e, (of, c) in enumerate(zip(offs, counts)):
        dY[of:of + c] = _rand(c, N, seed=30 + e)
    G = [torch.ones(N, K, dtype=torch.bfloat16, device="cuda") for _ in range(LE)]
    ep_fused._ragged_wgrad(dY, A, G, seg, LE, cap, N, K)
    torch.cuda.synchronize()
    for e, (of, c) in enumerate(zip(offs, counts)):
        want = 1.0 + dY[of:of + c].float().t() @ A[of:of + c].float()
        assert _rel_err(G[e], want) < 1e-2, (e, _rel_err(G[e], want))


def _tiny_moe(seed=0, dtype=torch.bfloat16):
    from lightron_b200 import mesh
    from lightron_b200.config import ModelArgs
    from lightron_b200.models import LightronTransformer, init_weights
    from lightron_b200.optim import DistributedAdamW
    mesh.set_context(None)
    args = ModelArgs(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=1024, intermediate_size=512,
                     max_seq_len=128, moe_num_experts=4, moe_topk=2, moe_layer_freq=1, moe_aux_loss_coef=0.01)
    model = LightronTransformer(args, dtype=torch.bfloat16, device=torch.device("cuda", 0))
    init_weights(model, seed)                       # bf16-rounded values, also for the fp32 oracle
    if dtype != torch.bfloat16:
        model = model.to(dtype)
    opt = DistributedAdamW(model, lr=1e-3)
    return model, opt, args


def _ff_grads(fused: bool, dtype=torch.bfloat16):
    """One MoE feed-forward on fixed inputs: output, aux loss and the gradients of the input, the
    gate and every expert weight."""
    from lightron_b200.models.moe import MoEFeedForward
    os.environ["LIGHTRON_FUSED_EP"] = "1" if fused else "0"
    try:
        model, opt, args = _tiny_moe(dtype=dtype)
        ff = next(b.feed_forward for b in model.layers.values() if isinstance(b.feed_forward, MoEFeedForward))
        x = _rand(256, args.dim, seed=3).to(dtype).requires_grad_(True)
        r = _rand(256, args.dim, seed=4).float()
        opt.zero_grad()
        y = ff(x)
        aux = ff.last_aux_loss
        ((y.float() * r).sum() + 3.0 * aux).backward()
        torch.cuda.synchronize()
        grads = {"x": x.grad.detach().float().clone()}
        grads.update({n: p.grad.detach().float().clone() for n, p in ff.named_parameters()})
        return y.detach().float(), float(aux), grads
    finally:
        os.environ.pop("LIGHTRON_FUSED_EP", None)


def test_fused_moe_matches_fp32_oracle():
    """Output, load-balance loss and every gradient of one MoE feed-forward (4 experts, top-2) on
    fixed inputs: the kernel chain (bf16) against the same module in fp32 on PyTorch ops, with the
    bf16 library-call path (argsort / index_select / all-to-all) measured next to it."""
    y_want, aux_want, g_want = _ff_grads(False, torch.float32)
    y_lib, aux_lib, g_lib = _ff_grads(False)
    y_k, aux_k, g_k = _ff_grads(True)
    assert _moe_status()[0] == 0
    assert _rel_err(y_k, y_want) < 1e-2, _rel_err(y_k, y_want)
    assert abs(aux_k - aux_want) < 1e-3 * max(1.0, abs(aux_want)), (aux_k, aux_want)
    for name, want in g_want.items():
        den = want.norm().clamp_min(1e-6)
        e_k = ((g_k[name] - want).norm() / den).item()
        e_lib = ((g_lib[name] - want).norm() / den).item()
        assert e_k < max(1.5 * e_lib, 2e-2), f"{name}: kernel chain {e_k:.4f} vs library path {e_lib:.4f}"


def test_fused_moe_drops_copies_beyond_capacity():
    """Expert-side buffers smaller than the routed load: the excess copies are dropped and counted, nothing is
    written out of bounds, nothing raises, and forward / backward stay finite."""
    from lightron_b200.models.moe import MoEFeedForward
    from lightron_b200.ops import native
    os.environ["LIGHTRON_FUSED_EP"] = "1"
    try:
        model, opt, args = _tiny_moe()
        ff = next(b.feed_forward for b in model.layers.values() if isinstance(b.feed_forward, MoEFeedForward))
        ff.capacity_factor = 0.25                         # 4096 routed copies, room for 1024 (+ 512 rows of padding)
        native.device_status(); native.take_moe_dropped()
        x = _rand(2048, args.dim, seed=3).requires_grad_(True)
        opt.zero_grad()
        y = ff(x)
        (y.float().sum() + ff.last_aux_loss).backward()
        torch.cuda.synchronize()
        assert not native.device_status()                 # a drop is not a failure
        dropped = native.take_moe_dropped()
        assert dropped["events"] > 0 and dropped["max_rows"] > 0
        assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all()
        kept = (y.float().abs().sum(dim=1) > 0).float().mean().item()
        assert 0.1 < kept < 1.0                           # tokens whose copies were all dropped give zero rows
        for p in ff.parameters():
            assert torch.isfinite(p.grad.float()).all()
    finally:
        os.environ.pop("LIGHTRON_FUSED_EP", None)


def test_fused_moe_model_step():
    """A whole small MoE model: the loss of the kernel-chain run agrees with the library-call run."""
    from lightron_b200.ops import native
    out = {}
    for fused in (False, True):
        os.environ["LIGHTRON_FUSED_EP"] = "1" if fused else "0"
        try:
            model, opt, args = _tiny_moe()
            g = torch.Generator(device="cuda").manual_seed(5)
            tok = torch.randint(0, args.vocab_size, (2, 128), device="cuda", generator=g)
            losses = []
            for _ in range(3):
                opt.zero_grad()
                loss = model.loss(tok, torch.roll(tok, -1, dims=1))
                loss.backward()
                opt.step()
                losses.append(float(loss.detach()))
            out[fused] = losses
        finally:
            os.environ.pop("LIGHTRON_FUSED_EP", None)
    assert not native.device_status()
    for a, b in zip(out[True], out[False]):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), out
    assert out[True][-1] < out[True][0]


def test_fused_moe_never_waits_on_the_host():
    """Forward + backward of the MoE feed-forward with synchronising calls turned into errors."""
    from lightron_b200.models.moe import MoEFeedForward
    model, opt, args = _tiny_moe()
    ff = next(b.feed_forward for b in model.layers.values() if isinstance(b.feed_forward, MoEFeedForward))
    x = _rand(256, args.dim, seed=3).requires_grad_(True)
    opt.zero_grad()
    y = ff(x)                                     # first call: buffers are allocated (may synchronise)
    (y.float().sum() + ff.last_aux_loss).backward()
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        x2 = x.detach().clone().requires_grad_(True)
        y = ff(x2)
        (y.float().sum() + ff.last_aux_loss).backward()
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    assert _moe_status()[0] == 0
    assert torch.isfinite(x2.grad.float()).all()
