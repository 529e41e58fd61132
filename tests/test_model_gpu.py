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
