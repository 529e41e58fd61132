"""End-to-end bf16 model on the native kernels against the fp32 PyTorch path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tiny_model_loss_and_grads_match_fp32_oracle():
    from lightron_b200 import mesh
    from lightron_b200.config import ModelArgs
    from lightron_b200.models import LightronTransformer, init_weights
    from lightron_b200.ops import native
    mesh.set_context(None)
    dev = torch.device("cuda", 0)
    args = ModelArgs(dim=256, n_layers=2, n_heads=8, n_kv_heads=4, vocab_size=2048, intermediate_size=688, max_seq_len=128)
    ref = LightronTransformer(args, dtype=torch.float32, device=dev)
    init_weights(ref, 0)
    m = LightronTransformer(args, dtype=torch.bfloat16, device=dev)
    m.load_state_dict({k: v.to(torch.bfloat16) for k, v in ref.state_dict().items()})
    ref.load_state_dict({k: v.float() for k, v in m.state_dict().items()})     # same rounded weights
    tok = torch.randint(0, args.vocab_size, (2, 128), device=dev)
    tgt = torch.randint(0, args.vocab_size, (2, 128), device=dev)
    n0 = native.launch_count()
    loss = m.loss(tok, tgt)
    loss.backward()
    assert native.launch_count() - n0 > 20          # the CUDA path ran, not a fallback
    lref = ref.loss(tok, tgt)
    lref.backward()
    assert abs(loss.item() - lref.item()) < 2e-2
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        err = (p.grad.float() - q.grad).norm() / q.grad.norm().clamp_min(1e-9)
        assert err < 6e-2, f"{n}: rel grad err {err.item()}"


def test_smoke_entry():
    import __graft_entry__ as g
    g.smoke()


def test_moe_grouped_expert_gemm_matches_per_expert_loop(monkeypatch):
    """A MoE model with four local experts: the grouped-GEMM expert path (parameters in the flat
    arena, weight gradients accumulated by the kernel) against the per-expert loop and the fp32 oracle."""
    from lightron_b200 import mesh
    from lightron_b200.config import ModelArgs
    from lightron_b200.models import LightronTransformer, init_weights
    from lightron_b200.ops import functional as OF, native
    from lightron_b200.optim import DistributedAdamW
    mesh.set_context(None)
    monkeypatch.setenv("LIGHTRON_FUSED_EP", "0")        # this test is about the library-exchange path (the kernel chain has its own)
    dev = torch.device("cuda", 0)
    args = ModelArgs(dim=256, n_layers=2, n_heads=8, n_kv_heads=4, vocab_size=1024, intermediate_size=512,
                     max_seq_len=128, moe_num_experts=4, moe_topk=2, moe_layer_freq=1)
    ref = LightronTransformer(args, dtype=torch.float32, device=dev)
    init_weights(ref, 1)
    g = torch.Generator().manual_seed(5)
    tok = torch.randint(0, args.vocab_size, (2, 128), generator=g).to(dev)
    tgt = torch.randint(0, args.vocab_size, (2, 128), generator=g).to(dev)
    results = {}
    for grouped in (True, False):
        m = LightronTransformer(args, dtype=torch.bfloat16, device=dev)
        m.load_state_dict({k: v.to(torch.bfloat16) for k, v in ref.state_dict().items()})
        opt = DistributedAdamW(m, lr=1e-3)              # builds the arena: w1 | w3 adjacent, grads preset
        if not grouped:
            monkeypatch.setattr(OF, "grouped_linear_ok", lambda *a, **k: False)
        opt.zero_grad()
        n0 = native.launch_count()
        loss = m.loss(tok, tgt)
        loss.backward()
        torch.cuda.synchronize()
        results[grouped] = (loss.item(), {n: p.grad.float().clone() for n, p in m.named_parameters()},
                            native.launch_count() - n0)
    ref.load_state_dict({k: v.float() for k, v in m.state_dict().items()})
    lref = ref.loss(tok, tgt)
    lref.backward()
    assert abs(results[True][0] - results[False][0]) < 1e-2 and abs(results[True][0] - lref.item()) < 3e-2
    assert results[True][2] < results[False][2]         # fewer launches with the grouped path
    gref = {n: p.grad for n, p in ref.named_parameters()}
    for n, g in results[True][1].items():
        other = results[False][1][n]
        err = (g - other).norm() / other.norm().clamp_min(1e-9)
        assert err < 3e-2, f"{n}: grouped vs loop rel grad err {err.item()}"
        err = (g - gref[n]).norm() / gref[n].norm().clamp_min(1e-9)
        # the router sees bf16 activations here and fp32 ones in the oracle: near-ties of the top-k
        # flip for a few tokens, which moves every gradient upstream of a MoE layer more than rounding
        # does; the tight check is the one against the per-expert loop above (same routing)
        assert err < 0.3, f"{n}: grouped vs fp32 rel grad err {err.item()}"
