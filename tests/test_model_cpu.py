import torch

from lightron_b200.config import ModelArgs, PRESETS
from lightron_b200.models import LightronTransformer, init_weights
from lightron_b200.optim import DistributedAdamW
from oracle import oracle_forward, oracle_loss


def _tiny(**kw):
    base = dict(PRESETS["tiny"])
    base.update(max_seq_len=64, n_layers=2)
    base.update(kw)
    return ModelArgs(**base)


def test_state_dict_keys_match_reference_layout():
    m = LightronTransformer(_tiny())
    keys = set(m.state_dict().keys())
    want = {"tok_embeddings.weight", "output.weight", "norm.weight"}
    for i in range(2):
        for n in ("wq", "wk", "wv", "wo"):
            want.add(f"layers.{i}.attention.{n}.weight")
        for n in ("w1", "w2", "w3"):
            want.add(f"layers.{i}.feed_forward.{n}.weight")
        want.add(f"layers.{i}.attention_norm.weight")
        want.add(f"layers.{i}.ffn_norm.weight")
    assert keys == want


def test_forward_matches_oracle_mha_and_gqa():
    for kv in (8, 2):
        a = _tiny(n_kv_heads=kv)
        m = LightronTransformer(a)
        init_weights(m, 1)
        tok = torch.randint(0, a.vocab_size, (2, 48))       # shorter than max_seq_len on purpose
        got = m(tok)
        want = oracle_forward(m.state_dict(), tok, n_layers=2, n_heads=8, n_kv_heads=kv)
        assert torch.allclose(got, want, atol=2e-5, rtol=1e-4), (got - want).abs().max()


def test_loss_and_grads_match_oracle():
    a = _tiny(n_kv_heads=4)
    m = LightronTransformer(a)
    init_weights(m, 2)
    tok = torch.randint(0, a.vocab_size, (2, 64))
    tgt = torch.randint(0, a.vocab_size, (2, 64))
    loss = m.loss(tok, tgt)
    loss.backward()
    sd = {k: v.detach().clone().requires_grad_(True) for k, v in m.state_dict().items()}
    ol = oracle_loss(sd, tok, tgt, n_layers=2, n_heads=8, n_kv_heads=4)
    ol.backward()
    assert abs(loss.item() - ol.item()) < 1e-5
    for name, p in m.named_parameters():
        assert torch.allclose(p.grad, sd[name].grad, atol=1e-6, rtol=1e-3), name


def test_moe_matches_dense_oracle():
    a = _tiny(moe_num_experts=4, moe_topk=2, moe_layer_freq=1, moe_aux_loss_coef=0.0)
    m = LightronTransformer(a)
    init_weights(m, 3)
    tok = torch.randint(0, a.vocab_size, (2, 32))
    got = m(tok)
    want = oracle_forward(m.state_dict(), tok, n_layers=2, n_heads=8, n_kv_heads=8)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-4)
    assert any("experts.3.w2.weight" in k for k in m.state_dict())


def test_adamw_matches_torch_optim():
    a = _tiny()
    m1 = LightronTransformer(a)
    init_weights(m1, 4)
    m2 = LightronTransformer(a)
    m2.load_state_dict(m1.state_dict())
    o1 = DistributedAdamW(m1, lr=3e-4, weight_decay=0.01)
    o2 = torch.optim.AdamW(m2.parameters(), lr=3e-4, weight_decay=0.01)
    g = torch.Generator().manual_seed(0)
    for _ in range(3):
        tok = torch.randint(0, a.vocab_size, (2, 64), generator=g)
        o1.zero_grad()
        o2.zero_grad()
        m1.loss(tok, tok).backward()
        m2.loss(tok, tok).backward()
        o1.step()
        o2.step()
    for (n, p1), (_, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.allclose(p1, p2, atol=1e-6), n


def test_flat_arena_makes_qkv_adjacent():
    from lightron_b200.ops.functional import _rows_adjacent
    a = _tiny(n_kv_heads=2)
    m = LightronTransformer(a)
    init_weights(m, 5)
    DistributedAdamW(m)
    att = m.layers["0"].attention
    assert _rows_adjacent((att.wq.weight, att.wk.weight, att.wv.weight))
    ff = m.layers["0"].feed_forward
    assert _rows_adjacent((ff.w1.weight, ff.w3.weight))
