"""Small, self-terminating workloads for profiling single kernels under ncu.

    python -m lightron_b200.profile_kernels gemm|grouped|normbwd|attn|norm|attn_full|mlp

Each mode launches its kernel a few times on inputs larger than L2 but well under 1 GB, prints
CUDA-event timings and exits; capture with e.g.
    ncu --set full --clock-control none -k regex:gemm_bf16 -s 2 -c 1 -o out python -m lightron_b200.profile_kernels gemm
``attn_full`` (the attention kernels at the 1.1 B and 8 B layer shapes next to the PyTorch library
attention) and ``mlp`` (the SwiGLU epilogues against GEMM + separate pass) are timing-only modes at full
size: CUDA events, not meant for ncu.
"""
from __future__ import annotations

import sys

import torch


def _time(fn, iters=5):
    for _ in range(2):
        fn()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record(); torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return sorted(ts)[len(ts) // 2]


def main(mode: str) -> None:
    from .ops import functional as OF
    dev = torch.device("cuda", 0)
    if mode == "gemm":
        M, N, K = 8192, 8192, 4096
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: OF.gemm(a, b))
        print(f"gemm {M}x{N}x{K}: {ms:.3f} ms  {2.0 * M * N * K / ms / 1e9:.0f} TFLOP/s")
    elif mode == "attn":
        B, S, hq, hkv, d = 4, 2048, 16, 4, 64
        q = torch.randn(B, S, hq, d, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, S, hkv, d, device=dev, dtype=torch.bfloat16)
        v = torch.randn(B, S, hkv, d, device=dev, dtype=torch.bfloat16)
        sc = d ** -0.5
        o, lse = OF.flash_fwd_native(q, k, v, True, sc)
        do = torch.randn_like(o)
        fl = 4.0 * B * hq * S * S * d / 2
        f = _time(lambda: OF.flash_fwd_native(q, k, v, True, sc))
        bw = _time(lambda: OF.flash_bwd_native(q, k, v, o, lse, do, True, sc))
        print(f"attention B{B} S{S} hq{hq} hkv{hkv} d{d}: fwd {f:.3f} ms {fl / f / 1e9:.0f} TFLOP/s, "
              f"bwd {bw:.3f} ms {2.5 * fl / bw / 1e9:.0f} TFLOP/s")
    elif mode == "norm":
        rows, cols = 65536, 2048                       # 256 MiB per tensor
        x = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16, requires_grad=True)
        r = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16)
        w = torch.ones(cols, device=dev, dtype=torch.bfloat16, requires_grad=True)
        ms = _time(lambda: OF.add_rmsnorm(x, r, w, 1e-5))
        gb = 4 * rows * cols * 2 / 1e9
        print(f"add_rmsnorm fwd {rows}x{cols}: {ms:.3f} ms  {gb / ms * 1e3:.0f} GB/s")
    elif mode == "grouped":
        # data gradient of the 1.1B model's gate+up projection: plain kernel, grouped kernel with
        # that one problem, then the layer's data + weight gradient as one grouped launch
        T, N, K = 16384, 11264, 2048
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(T, N, device=dev, dtype=torch.bfloat16)
        fl = 2.0 * T * N * K
        t_plain = _time(lambda: OF.gemm(dy, w, b_mn=True, legacy=True), iters=3)
        t_one = _time(lambda: OF.gemm_grouped([(dy, w, False, True, None, False)]), iters=3)
        t_w = _time(lambda: OF.gemm(dy, x, a_mn=True, b_mn=True, legacy=True), iters=3)
        t_pair = _time(lambda: OF.gemm_grouped([(dy, x, True, True, None, False), (dy, w, False, True, None, False)]),
                       iters=3)
        print(f"dgrad {T}x{K}x{N}: plain {t_plain:.3f} ms ({fl / t_plain / 1e9:.0f} TFLOP/s), grouped(1) {t_one:.3f} ms "
              f"({fl / t_one / 1e9:.0f}); plain wgrad {t_w:.3f} ms; dgrad+wgrad grouped {t_pair:.3f} ms "
              f"({2 * fl / t_pair / 1e9:.0f} TFLOP/s) vs {t_plain + t_w:.3f} ms separate")
    elif mode == "normbwd":
        rows, cols = 32768, 2048                       # 128 MiB per tensor
        x = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16, requires_grad=True)
        r = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = torch.ones(cols, device=dev, dtype=torch.bfloat16, requires_grad=True)
        h, y = OF.add_rmsnorm(x, r, w, 1e-5)
        dh, dyy = torch.randn_like(h), torch.randn_like(y)
        ms = _time(lambda: torch.autograd.grad([h, y], [x, r, w], [dh, dyy], retain_graph=True), iters=3)
        gb = 4 * rows * cols * 2 / 1e9                 # dy, x, dres in; dx out (dx doubles as the residual gradient)
        print(f"add_rmsnorm bwd {rows}x{cols}: {ms:.3f} ms  {gb / ms * 1e3:.0f} GB/s (autograd call, both kernels)")
    elif mode == "attn_full":
        import torch.nn.functional as F
        for (B, S, hq, hkv, d) in [(8, 2048, 32, 4, 64), (1, 8192, 32, 8, 128), (2, 4096, 16, 16, 64)]:
            q = torch.randn(B, S, hq, d, device=dev, dtype=torch.bfloat16)
            k = torch.randn(B, S, hkv, d, device=dev, dtype=torch.bfloat16)
            v = torch.randn(B, S, hkv, d, device=dev, dtype=torch.bfloat16)
            fl = 4.0 * B * hq * S * S * d / 2
            sc = d ** -0.5
            t_f = _time(lambda: OF.flash_fwd_native(q, k, v, True, sc), iters=10)
            o, lse = OF.flash_fwd_native(q, k, v, True, sc)
            do = torch.randn_like(o)
            t_b = _time(lambda: OF.flash_bwd_native(q, k, v, o, lse, do, True, sc), iters=10)
            # the library attention the reference calls (model/model.py:193-198), K / V expanded to the query heads
            qt = q.transpose(1, 2)
            kt, vt = (t.transpose(1, 2).repeat_interleave(hq // hkv, 1) for t in (k, v))
            t_lib = _time(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True), iters=10)
            qr, kr, vr = (t.clone().requires_grad_(True) for t in (qt, kt, vt))

            def lib_fb():
                F.scaled_dot_product_attention(qr, kr, vr, is_causal=True).backward(do.transpose(1, 2))
            t_lib_fb = _time(lib_fb, iters=10)
            print(f"B{B} S{S} hq{hq} hkv{hkv} d{d}: fwd {t_f:.3f} ms {fl / t_f / 1e9:.0f} TFLOP/s | bwd {t_b:.3f} ms "
                  f"{2.5 * fl / t_b / 1e9:.0f} TFLOP/s | library fwd {t_lib:.3f} ms {fl / t_lib / 1e9:.0f} TFLOP/s, "
                  f"fwd+bwd {t_lib_fb:.3f} ms", flush=True)
    elif mode == "mlp":
        from .ops import native
        T, K, I = 16384, 2048, 5632
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        w13 = torch.randn(2 * I, K, device=dev, dtype=torch.bfloat16) * 0.02
        w2 = torch.randn(K, I, device=dev, dtype=torch.bfloat16) * 0.02
        dy = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        gu = torch.empty(T, 2 * I, device=dev, dtype=torch.bfloat16)
        h = torch.empty(T, I, device=dev, dtype=torch.bfloat16)
        dgu, dh = torch.empty_like(gu), torch.empty_like(h)
        dw2 = torch.zeros(K, I, device=dev, dtype=torch.bfloat16)
        st = native.stream_ptr
        t_g = _time(lambda: OF.gemm_grouped([(x, w13, False, False, gu, False)]), iters=10)
        t_s = _time(lambda: native.call("lb_swiglu_fwd", gu.data_ptr(), h.data_ptr(), T, I, gu.stride(0), st()), iters=10)
        t_e = _time(lambda: OF.gemm_grouped([(x, w13, False, False, gu, False, 1, h, I)]), iters=10)
        print(f"gate | up GEMM {t_g:.3f} ms + SwiGLU pass {t_s:.3f} ms = {t_g + t_s:.3f} ms | with the epilogue {t_e:.3f} ms")
        t_p = _time(lambda: OF.gemm_grouped([(dy, h, True, True, dw2, True), (dy, w2, False, True, dh, False)]), iters=10)
        t_sb = _time(lambda: native.call("lb_swiglu_bwd", gu.data_ptr(), dh.data_ptr(), dgu.data_ptr(), T, I, gu.stride(0), st()),
                     iters=10)
        t_pe = _time(lambda: OF.gemm_grouped([(dy, h, True, True, dw2, True), (dy, w2, False, True, dgu, False, 2, gu, I)]),
                     iters=10)
        print(f"[weight + data gradient of down] {t_p:.3f} ms + SwiGLU-backward pass {t_sb:.3f} ms = {t_p + t_sb:.3f} ms | "
              f"with the epilogue {t_pe:.3f} ms")
    else:
        raise SystemExit("mode: gemm | grouped | normbwd | attn | norm | attn_full | mlp")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "gemm")
