"""Independent single-device fp32 restatement of the reference model math (complex RoPE,
SDPA with repeated KV), used as the numeric oracle.  Mirrors model/model.py and layers/layers.py
of the reference, with the GQA view fixed."""
import math

import torch
import torch.nn.functional as F


def oracle_forward(sd, tokens, n_layers, n_heads, n_kv_heads, eps=1e-5, theta=10000.0):
    x = F.embedding(tokens, sd["tok_embeddings.weight"])
    B, S, H = x.shape
    d = H // n_heads
    freqs = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
    ang = torch.outer(torch.arange(S).float(), freqs)
    fc = torch.polar(torch.ones_like(ang), ang).view(1, S, 1, d // 2)

    def norm(t, w):
        tf = t.float()
        return (tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + eps)).type_as(t) * w

    def rot(t):
        tc = torch.view_as_complex(t.float().reshape(*t.shape[:-1], -1, 2))
        return torch.view_as_real(tc * fc).flatten(3).type_as(t)

    for i in range(n_layers):
        p = f"layers.{i}."
        h = norm(x, sd[p + "attention_norm.weight"])
        q = F.linear(h, sd[p + "attention.wq.weight"]).view(B, S, n_heads, d)
        k = F.linear(h, sd[p + "attention.wk.weight"]).view(B, S, n_kv_heads, d)
        v = F.linear(h, sd[p + "attention.wv.weight"]).view(B, S, n_kv_heads, d)
        q, k = rot(q), rot(k)
        rep = n_heads // n_kv_heads
        k = k.repeat_interleave(rep, dim=2)
        v = v.repeat_interleave(rep, dim=2)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        o = o.transpose(1, 2).reshape(B, S, -1)
        x = x + F.linear(o, sd[p + "attention.wo.weight"])
        h = norm(x, sd[p + "ffn_norm.weight"])
        if p + "feed_forward.w1.weight" in sd:
            f = F.linear(F.silu(F.linear(h, sd[p + "feed_forward.w1.weight"])) * F.linear(h, sd[p + "feed_forward.w3.weight"]),
                         sd[p + "feed_forward.w2.weight"])
        else:
            f = oracle_moe(sd, p + "feed_forward.", h)
        x = x + f
    x = norm(x, sd["norm.weight"])
    return F.linear(x, sd["output.weight"])


def oracle_moe(sd, p, h, topk=2):
    B, S, H = h.shape
    x = h.reshape(-1, H)
    probs = F.softmax(F.linear(x, sd[p + "gate.weight"]).float(), dim=-1)
    w, idx = torch.topk(probs, topk, dim=-1)
    out = torch.zeros_like(x)
    E = probs.shape[-1]
    for e in range(E):
        fe = F.linear(F.silu(F.linear(x, sd[p + f"experts.{e}.w1.weight"])) * F.linear(x, sd[p + f"experts.{e}.w3.weight"]),
                      sd[p + f"experts.{e}.w2.weight"])
        for kk in range(topk):
            m = (idx[:, kk] == e).float().unsqueeze(-1)
            out = out + m * w[:, kk:kk + 1] * fe
    return out.view(B, S, H)


def oracle_loss(sd, tokens, targets, **kw):
    logits = oracle_forward(sd, tokens, **kw)
    return F.cross_entropy(logits.view(-1, logits.size(-1)), targets.view(-1))
